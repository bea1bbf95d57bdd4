// Long-implicit (HCL) Hyena operator: y = x2 * (h * u + D u) with
// u = bf16(x1 * v) and the per-channel modal filter
// h[c,t] = sum_m R[c,m] exp(log_pole[c,m] t).
//
// Upstream materialises h and convolves with an n = 2T FFT, then recovers the
// decode state with one complex FFT per (channel, mode)
// (src/cuda/hyena.cu:562-660, 1262-1456, 1994-2124).  Because the filter is a
// sum of first-order modes, the same convolution is a linear recurrence
// s_m[t] = p_m s_m[t-1] + u[t], y[t] = sum_m R_m s_m[t]; here it runs as a
// two-kernel chunked scan that is linear in T, needs one state per segment of
// scratch instead of FFT planes, and yields the decode state for free:
//   1. per (segment, channel pair): end state of the segment from zero,
//   2. per (segment, channel pair): fold the end states of the earlier
//      segments into the carried-in state (p^S scaling), replay from it, read
//      out, add the direct term, post-gate, store.
// The four BF16 roundings of the upstream epilogue are kept for initial
// prefill; continuation chunks keep upstream's single rounding
// (src/cuda/hyena.cu:534-560).  modal_decode keeps the pinned decode order
// (separate multiply/add, 32-lane zero-padded tree; src/cuda/hyena.cu:718-761).
#include <algorithm>
#include <cstdlib>
#include <mutex>
#include <string>
#include <type_traits>

#include "common.cuh"
#include "ops_internal.hpp"
#include "projection_featurizer.cuh"

namespace evob {
namespace {

struct ModalParams {
  const bf16 *x2, *x1, *value, *projection, *short_filter, *direct;
  const float *log_poles, *residues;
  bf16 *output, *pregate;
  float *state;    // [width, modes]
  float *scratch;  // [segments + 1, width, modes]
  float *short_cache;          // optional F32 [3 width, 2] raw projection history for decode
  std::size_t scratch_floats;  // capacity of scratch
  int length, row_begin, width, segment, segments, pairs;
  bool continue_from_state;
};

// One decode step of the modal recurrence.  A warp owns a channel and lane m
// its mode m: the state update is a separate multiply and add, the read-out
// terms R_m s_m sit in lanes 0..modes-1 of a zero-padded 32-lane shuffle-down
// fold - upstream's pinned order (src/cuda/hyena.cu:718-761) is literally a
// warp reduction, so the lanes are the reduction slots.
constexpr int kDecodeThreads = 256;

__global__ void __launch_bounds__(kDecodeThreads)
modal_decode_warp_kernel(const bf16 *__restrict__ x2, const bf16 *__restrict__ x1, const bf16 *__restrict__ value,
                         const bf16 *__restrict__ direct, const float *__restrict__ log_poles,
                         const float *__restrict__ residues, float *__restrict__ state, bf16 *__restrict__ pregate,
                         bf16 *__restrict__ output, const int width, const int modes) {
  const int channel = (blockIdx.x * kDecodeThreads + threadIdx.x) / 32;
  const int lane = threadIdx.x % 32;
  if (channel >= width) return;
  const float gated = rbf(bf2f(x1[channel]) * bf2f(value[channel]));
  float term = 0.0F;
  if (lane < modes) {
    const std::size_t q = static_cast<std::size_t>(channel) * modes + lane;
    const float updated = __fadd_rn(__fmul_rn(expf(log_poles[q]), state[q]), gated);
    state[q] = updated;
    term = __fmul_rn(residues[q], updated);
  }
#pragma unroll
  for (int offset = 16; offset != 0; offset /= 2) {
    const float other = __shfl_down_sync(0xffffffffU, term, offset);
    if (lane < 32 - offset) term = __fadd_rn(term, other);
  }
  if (lane != 0) return;
  if (pregate != nullptr) pregate[channel] = f2bf(gated);
  const float direct_product = rbf(bf2f(direct[channel]) * gated);
  output[channel] = f2bf(__fmul_rn(bf2f(x2[channel]), __fadd_rn(term, direct_product)));
}

// Diagnostic taps of the long-implicit operator (upstream's kMixerFilter and
// kMixerConvolution dump points, src/cuda/model.cu:1570-1581): the time-domain
// filter h[t, c] with upstream's four-accumulator mode sum
// (src/cuda/hyena.cu:562-592) and the F32 convolution y[t, c] = sum_s h[t-s] u[s]
// before any rounding, evaluated as the modal recurrence from a zero state.
// Thread = channel, walking time; neighbouring threads write neighbouring
// columns of the [length, width] outputs.
__global__ void modal_taps_kernel(const bf16 *__restrict__ gated, const float *__restrict__ log_poles,
                                  const float *__restrict__ residues, float *__restrict__ filter,
                                  float *__restrict__ convolution, const int length, const int width,
                                  const int modes) {
  const int channel = blockIdx.x * blockDim.x + threadIdx.x;
  if (channel >= width) return;
  const float *const lp = log_poles + static_cast<std::size_t>(channel) * modes;
  const float *const res = residues + static_cast<std::size_t>(channel) * modes;
  float state[32];
#pragma unroll
  for (int m = 0; m < 32; ++m) state[m] = 0.0F;
  for (int t = 0; t < length; ++t) {
    const std::size_t at = static_cast<std::size_t>(t) * width + channel;
    if (filter != nullptr) {
      float partial[4] = {0.0F, 0.0F, 0.0F, 0.0F};
      for (int m = 0; m < modes; ++m)
        partial[m % 4] = __fadd_rn(partial[m % 4], __fmul_rn(res[m], expf(lp[m] * static_cast<float>(t))));
      filter[at] = __fadd_rn(__fadd_rn(__fadd_rn(partial[0], partial[1]), partial[2]), partial[3]);
    }
    if (convolution != nullptr) {
      const float u = bf2f(gated[at]);
      float y = 0.0F;
#pragma unroll
      for (int m = 0; m < 32; ++m) {
        if (m < modes) {
          state[m] = fmaf(expf(lp[m]), state[m], u);
          y = fmaf(res[m], state[m], y);
        }
      }
      convolution[at] = y;
    }
  }
}

// -------------------------------------------------------- register streaming
// Two kernels, no shared memory.  A thread owns one channel pair and walks down
// one segment of rows with the featurizer history, the poles and the 2 x modes
// states in registers; the loads of the next kUnroll rows are in flight while
// the current ones are consumed, so every input element is read once per pass
// with nothing staged.  The grid is one wave: as many segments as fill every SM
// once.
//   pass 1 (kOutput = false)  end state of each segment but the last, from zero
//   pass 2 (kOutput = true)   every thread first folds the end states of the
//                             segments before its own into its carried-in state
//                             (a serial chain of at most `segments` steps per
//                             mode), then replays its segment, reads out, applies
//                             the epilogue and stores; the thread of the last
//                             segment leaves the decode state and the featurizer
//                             history behind.
// scratch: [segments] local end states, then one slot for the state carried into
// the first segment of a continuation (copied there by pass 1, because pass 2
// overwrites p.state while other segments may still have to read it).
constexpr int kStreamThreads = 128;

__device__ __forceinline__ std::uint32_t mul_pairs(const std::uint32_t a, const std::uint32_t b) {
  std::uint32_t d;  // both products rounded once: the bits of rbf(float(a) * float(b))
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ std::uint32_t add_pairs(const std::uint32_t a, const std::uint32_t b) {
  std::uint32_t d;  // sums of BF16 values rounded once: the bits of rbf(float(a) + float(b))
  asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ float pair_lo(const std::uint32_t w) { return __uint_as_float(w << 16U); }
__device__ __forceinline__ float pair_hi(const std::uint32_t w) { return __uint_as_float(w & 0xffff0000U); }

// Two F32 values in one 64-bit register and the packed FMA of sm_100 on them: each half is an
// ordinary round-to-nearest FMA, so a pair of modes advanced this way has the bits of two scalar FMAs.
__device__ __forceinline__ unsigned long long pack_f32_pair(const float low, const float high) {
  unsigned long long pair;
  asm("mov.b64 %0, {%1, %2};" : "=l"(pair) : "f"(low), "f"(high));
  return pair;
}
__device__ __forceinline__ void unpack_f32_pair(const unsigned long long pair, float &low, float &high) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(low), "=f"(high) : "l"(pair));
}
__device__ __forceinline__ unsigned long long fma_f32_pair(const unsigned long long a, const unsigned long long b,
                                                           const unsigned long long c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}

// kC = 2: a channel pair per thread, one 32-bit word per stream and row.  kC = 1: one channel per
// thread with the same packed arithmetic on the low half of every word (the high half carries
// zeros), so a channel's bits do not depend on the form; half the registers, twice the warps.
template <int kModes, bool kProj, bool kOutput, int kUnroll, int kC>
__global__ void __launch_bounds__(kStreamThreads, kC == 1 ? (kOutput ? 4 : 5) : (kOutput ? 2 : 3))
modal_stream_kernel(const ModalParams p) {
  constexpr int kColumns = 3 * kC;  // projection-fed: (x2, x1, v) per channel; else x1 | v | x2
  const int c0 = (blockIdx.x * kStreamThreads + threadIdx.x) * kC;
  if (c0 >= p.width) return;
  const int seg = blockIdx.y;
  const int t_own = p.row_begin + seg * p.segment;
  const int t_end = min(p.length, t_own + p.segment);
  const std::size_t per_segment = static_cast<std::size_t>(p.width) * kModes;
  const std::size_t mine = static_cast<std::size_t>(c0) * kModes;  // the thread's kC x kModes values are contiguous

  float pole[kC][kModes], state[kC][kModes];
  [[maybe_unused]] float residue[kC][kModes];
  if constexpr (kOutput) {
    const float *const initial =
        p.continue_from_state ? (p.segments > 1 ? p.scratch + p.segments * per_segment : p.state) : nullptr;
#pragma unroll
    for (int c = 0; c < kC; ++c)
#pragma unroll
      for (int m = 0; m < kModes; ++m)
        state[c][m] = initial != nullptr ? __ldcg(initial + mine + c * kModes + m) : 0.0F;
    if (seg > 0) {
      float decay[kC][kModes];
#pragma unroll
      for (int c = 0; c < kC; ++c)
#pragma unroll
        for (int m = 0; m < kModes; ++m)
          decay[c][m] = expf(p.log_poles[mine + c * kModes + m] * static_cast<float>(p.segment));
      // The chain over segments is serial, its loads are not: four segments' end states are
      // requested before the first dependent FMA, so the fold costs seg / 4 round trips to L2.
      constexpr int kAhead = 4;
      for (int j0 = 0; j0 < seg; j0 += kAhead) {
        float local[kAhead][kC * kModes];
#pragma unroll
        for (int i = 0; i < kAhead; ++i) {
          const float *const source = p.scratch + (j0 + i) * per_segment + mine;
#pragma unroll
          for (int q = 0; q < kC * kModes; ++q) local[i][q] = j0 + i < seg ? __ldcg(source + q) : 0.0F;
        }
#pragma unroll
        for (int i = 0; i < kAhead; ++i) {
          if (j0 + i < seg) {
#pragma unroll
            for (int c = 0; c < kC; ++c)
#pragma unroll
              for (int m = 0; m < kModes; ++m)
                state[c][m] = fmaf(decay[c][m], state[c][m], local[i][c * kModes + m]);
          }
        }
      }
    }
  } else {
    if (seg == 0 && p.continue_from_state) {
      float *const slot = p.scratch + p.segments * per_segment + mine;
#pragma unroll
      for (int i = 0; i < kC * kModes; ++i) slot[i] = p.state[mine + i];
    }
#pragma unroll
    for (int c = 0; c < kC; ++c)
#pragma unroll
      for (int m = 0; m < kModes; ++m) state[c][m] = 0.0F;
  }
#pragma unroll
  for (int c = 0; c < kC; ++c)
#pragma unroll
    for (int m = 0; m < kModes; ++m) {
      pole[c][m] = expf(p.log_poles[mine + c * kModes + m]);
      if constexpr (kOutput) residue[c][m] = p.residues[mine + c * kModes + m];
    }
  [[maybe_unused]] std::uint32_t direct_pair = 0U;
  [[maybe_unused]] float direct[kC] = {};
  if constexpr (kOutput) {
    if constexpr (kC == 2) direct_pair = *reinterpret_cast<const std::uint32_t *>(p.direct + c0);
    else direct_pair = *reinterpret_cast<const unsigned short *>(p.direct + c0);
    direct[0] = pair_lo(direct_pair);
    if constexpr (kC == 2) direct[1] = pair_hi(direct_pair);
  }

  struct Row {
    // kC = 2, projection-fed: (x2a x1a) (va x2b) (x1b vb); separate inputs: x1 | v | x2 pairs.
    // kC = 1, projection-fed: the two words that hold the channel's three columns - an even channel
    // owns (x2 x1) (v .), an odd one (. x2) (x1 v); separate inputs: x1 | v | x2 in the low halves.
    std::uint32_t w[3];
  };
  [[maybe_unused]] const int odd = c0 & 1;  // kC = 1: which half of the channel pair's six columns
  const auto load_words = [&](Row &row, const int t, auto loader) {
    if constexpr (kProj) {
      const bf16 *const source = p.projection + static_cast<std::size_t>(t) * 3 * p.width +
                                 static_cast<std::size_t>(kC == 2 ? c0 : c0 - odd) * 3;
      if constexpr (kC == 2) {
#pragma unroll
        for (int i = 0; i < 3; ++i) row.w[i] = loader(reinterpret_cast<const unsigned int *>(source) + i);
      } else {
        row.w[0] = loader(reinterpret_cast<const unsigned int *>(source) + odd);
        row.w[1] = loader(reinterpret_cast<const unsigned int *>(source) + odd + 1);
      }
    } else {
      const std::size_t index = static_cast<std::size_t>(t) * p.width + c0;
      if constexpr (kC == 2) {
        row.w[0] = loader(reinterpret_cast<const unsigned int *>(p.x1 + index));
        row.w[1] = loader(reinterpret_cast<const unsigned int *>(p.value + index));
        if constexpr (kOutput) row.w[2] = loader(reinterpret_cast<const unsigned int *>(p.x2 + index));
      } else {
        row.w[0] = loader(reinterpret_cast<const unsigned short *>(p.x1 + index));
        row.w[1] = loader(reinterpret_cast<const unsigned short *>(p.value + index));
        if constexpr (kOutput) row.w[2] = loader(reinterpret_cast<const unsigned short *>(p.x2 + index));
      }
    }
  };
  const auto load_row = [&](auto checked, const int t) {
    constexpr bool kChecked = decltype(checked)::value;
    Row row;
    row.w[0] = row.w[1] = row.w[2] = 0U;
    if constexpr (kChecked) {
      if (t < 0 || t >= t_end) return row;
    }
    load_words(row, t, [](const auto *address) { return static_cast<std::uint32_t>(__ldcs(address)); });
    return row;
  };
  // The streaming loads walk the rows in order: the projection-fed form keeps a word pointer that moves
  // one row per call instead of rebuilding the 64-bit address from the row number.
  [[maybe_unused]] const unsigned int *cursor = nullptr;
  [[maybe_unused]] const std::size_t cursor_stride = static_cast<std::size_t>(p.width) * 3 / 2;  // words per row
  if constexpr (kProj)
    cursor = reinterpret_cast<const unsigned int *>(p.projection + static_cast<std::size_t>(t_own) * 3 * p.width +
                                                    static_cast<std::size_t>(kC == 2 ? c0 : c0 - odd) * 3) +
             (kC == 2 ? 0 : odd);
  const auto load_next_row = [&](auto checked, const int t) {
    if constexpr (!kProj) {
      return load_row(checked, t);
    } else {
      constexpr bool kChecked = decltype(checked)::value;
      Row row;
      row.w[0] = row.w[1] = row.w[2] = 0U;
      const unsigned int *const at = cursor;
      cursor += cursor_stride;
      if constexpr (kChecked) {
        if (t < 0 || t >= t_end) return row;
      }
      row.w[0] = __ldcs(at);
      row.w[1] = __ldcs(at + 1);
      if constexpr (kC == 2) row.w[2] = __ldcs(at + 2);
      return row;
    }
  };
  // projection-fed rows as one F32 value per column
  const auto columns_of = [&](const Row &row, float (&x)[kColumns]) {
    if constexpr (kC == 2) {
#pragma unroll
      for (int w = 0; w < 3; ++w) {
        x[2 * w] = pair_lo(row.w[w]);
        x[2 * w + 1] = pair_hi(row.w[w]);
      }
    } else {
      // even: lo(w0) hi(w0) lo(w1); odd: hi(w0) lo(w1) hi(w1)
      const std::uint32_t end_selector = odd ? 0x3244U : 0x1044U;  // byte_perm(w, 0, .): hi(w) or lo(w) as F32 bits
      x[0] = __uint_as_float(__byte_perm(row.w[0], 0U, end_selector));
      x[1] = __uint_as_float(__byte_perm(row.w[0], row.w[1], odd ? 0x5444U : 0x3244U) & 0xffff0000U);
      x[2] = __uint_as_float(__byte_perm(row.w[1], 0U, end_selector));
    }
  };
  constexpr std::true_type kCheckedRows{};
  constexpr std::false_type kPlainRows{};

  // featurizer: taps [column][tap] of the thread's columns, raw rows t-2 and t-1
  [[maybe_unused]] float st[kColumns][3], xh[2][kColumns];
  if constexpr (kProj) {
#pragma unroll
    for (int i = 0; i < kColumns * 3; ++i)
      st[i / 3][i % 3] = bf2f(p.short_filter[static_cast<std::size_t>(c0) * 9 + i]);
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      // t_end only bounds rows behind the segment; these lie in front of it
      const int t = t_own - 2 + k;
      Row row;
      row.w[0] = row.w[1] = row.w[2] = 0U;
      if (t >= 0) load_words(row, t, [](const auto *address) { return static_cast<std::uint32_t>(__ldg(address)); });
      columns_of(row, xh[k]);
    }
  }

  // One channel per thread, an even number of modes: the modes advance two at a time in packed
  // registers (pole, state and residue pairs); the scalar arrays are only the prologue's and the
  // epilogue's view of the same values.
  constexpr bool kPacked = kC == 1 && kModes % 2 == 0;
  constexpr int kPairs = kPacked ? kModes / 2 : 1;
  [[maybe_unused]] unsigned long long pole2[kPairs], state2[kPairs], residue2[kPairs];
  if constexpr (kPacked) {
#pragma unroll
    for (int q = 0; q < kPairs; ++q) {
      pole2[q] = pack_f32_pair(pole[0][2 * q], pole[0][2 * q + 1]);
      state2[q] = pack_f32_pair(state[0][2 * q], state[0][2 * q + 1]);
      if constexpr (kOutput) residue2[q] = pack_f32_pair(residue[0][2 * q], residue[0][2 * q + 1]);
    }
  }

  Row next[kUnroll];
  [[maybe_unused]] std::size_t out_offset = static_cast<std::size_t>(t_own) * p.width + c0;
  const auto run_group = [&](auto checked, const int base) {
    constexpr bool kChecked = decltype(checked)::value;
    Row rows[kUnroll];
#pragma unroll
    for (int i = 0; i < kUnroll; ++i) rows[i] = next[i];
#pragma unroll
    for (int i = 0; i < kUnroll; ++i) {
      const int t = base + i;
      // one row's loads per row of arithmetic instead of a burst of kUnroll rows: the
      // load / store queue of the SM is not flooded at the start of every group
      next[i] = load_next_row(checked, base + kUnroll + i);
      if (kChecked && t >= t_end) break;
      std::uint32_t u_pair;  // u and the x2 gate of the pair, packed BF16
      [[maybe_unused]] std::uint32_t gate_pair = 0U;
      if constexpr (kProj) {
        float x[kColumns], z[kColumns];
        columns_of(rows[i], x);
#pragma unroll
        for (int column = 0; column < kColumns; ++column) {
          if (!kOutput && column % 3 == 0) continue;  // the x2 gate is not needed for the state
          // fmaf with +0, not a multiply: the sign of a zero result must match the FMA chain
          float acc = fmaf(xh[0][column], st[column][0], 0.0F);
          acc = fmaf(xh[1][column], st[column][1], acc);
          z[column] = fmaf(x[column], st[column][2], acc);
          xh[0][column] = xh[1][column];
          xh[1][column] = x[column];
        }
        if constexpr (kC == 2) {
          if constexpr (kOutput) gate_pair = round_pair_bf16(z[0], z[3]);
          u_pair = mul_pairs(round_pair_bf16(z[1], z[4]), round_pair_bf16(z[2], z[5]));
        } else {
          if constexpr (kOutput) gate_pair = round_pair_bf16(z[0], 0.0F);
          u_pair = mul_pairs(round_pair_bf16(z[1], 0.0F), round_pair_bf16(z[2], 0.0F));
        }
      } else {
        u_pair = mul_pairs(rows[i].w[0], rows[i].w[1]);
        gate_pair = rows[i].w[2];
      }
      float u[kC];
      u[0] = pair_lo(u_pair);
      if constexpr (kC == 2) u[1] = pair_hi(u_pair);
      if constexpr (!kOutput) {
        if constexpr (kPacked) {
          const unsigned long long u2 = pack_f32_pair(u[0], u[0]);
#pragma unroll
          for (int q = 0; q < kPairs; ++q) state2[q] = fma_f32_pair(pole2[q], state2[q], u2);
        } else {
#pragma unroll
          for (int m = 0; m < kModes; ++m)
#pragma unroll
            for (int c = 0; c < kC; ++c) state[c][m] = fmaf(pole[c][m], state[c][m], u[c]);
        }
      } else {
        float modal[kC];
        if constexpr (kPacked) {
          // partial sums by mode % 4 as in the scalar form: pair q feeds (partial[0], partial[1]) when
          // q is even and (partial[2], partial[3]) when it is odd
          const unsigned long long u2 = pack_f32_pair(u[0], u[0]);
          unsigned long long partial2[2] = {0ULL, 0ULL};
#pragma unroll
          for (int q = 0; q < kPairs; ++q) {
            state2[q] = fma_f32_pair(pole2[q], state2[q], u2);
            partial2[q % 2] = fma_f32_pair(residue2[q], state2[q], partial2[q % 2]);
          }
          float partial[4];
          unpack_f32_pair(partial2[0], partial[0], partial[1]);
          unpack_f32_pair(partial2[1], partial[2], partial[3]);
          modal[0] = ((partial[0] + partial[1]) + partial[2]) + partial[3];
        } else {
#pragma unroll
          for (int c = 0; c < kC; ++c) {
            float partial[4] = {0.0F, 0.0F, 0.0F, 0.0F};
#pragma unroll
            for (int m = 0; m < kModes; ++m) {
              state[c][m] = fmaf(pole[c][m], state[c][m], u[c]);
              partial[m % 4] = fmaf(residue[c][m], state[c][m], partial[m % 4]);
            }
            modal[c] = ((partial[0] + partial[1]) + partial[2]) + partial[3];
          }
        }
        const std::size_t offset = out_offset;  // = t * width + c0, carried from row to row
        out_offset += static_cast<std::size_t>(p.width);
        std::uint32_t result;
        const float modal_high = kC == 2 ? modal[kC - 1] : 0.0F;
        if (p.continue_from_state) {
          result = pack_bf16x2(pair_lo(gate_pair) * fmaf(direct[0], u[0], modal[0]),
                               kC == 2 ? pair_hi(gate_pair) * fmaf(direct[kC - 1], u[kC - 1], modal_high) : 0.0F);
        } else {
          // bf16(bf16(bf16(modal) + bf16(D u)) x2), each step one rounding of an exact result
          const std::uint32_t mixed =
              add_pairs(round_pair_bf16(modal[0], modal_high), mul_pairs(direct_pair, u_pair));
          result = mul_pairs(mixed, gate_pair);
        }
        if constexpr (kC == 2) {
          *reinterpret_cast<std::uint32_t *>(p.output + offset) = result;
          if (p.pregate != nullptr) *reinterpret_cast<std::uint32_t *>(p.pregate + offset) = u_pair;
        } else {
          *reinterpret_cast<unsigned short *>(p.output + offset) = static_cast<unsigned short>(result);
          if (p.pregate != nullptr)
            *reinterpret_cast<unsigned short *>(p.pregate + offset) = static_cast<unsigned short>(u_pair);
        }
        if constexpr (kChecked && kProj) {
          // raw rows length-2 and length-1 are the featurizer's decode history
          if (p.short_cache != nullptr && t == p.length - 1) {
#pragma unroll
            for (int column = 0; column < kColumns; ++column)
              *reinterpret_cast<float2 *>(p.short_cache + (static_cast<std::size_t>(c0) * 3 + column) * 2) =
                  make_float2(xh[0][column], xh[1][column]);
          }
        }
      }
    }
  };

#pragma unroll
  for (int i = 0; i < kUnroll; ++i) next[i] = load_next_row(kCheckedRows, t_own + i);
  int base = t_own;
  for (; base + 2 * kUnroll <= t_end; base += kUnroll) run_group(kPlainRows, base);
  for (; base < t_end; base += kUnroll) run_group(kCheckedRows, base);
  if constexpr (kPacked) {
#pragma unroll
    for (int q = 0; q < kPairs; ++q) unpack_f32_pair(state2[q], state[0][2 * q], state[0][2 * q + 1]);
  }

  if constexpr (kOutput) {
    if (t_end == p.length && p.state != nullptr) {
#pragma unroll
      for (int c = 0; c < kC; ++c)
#pragma unroll
        for (int m = 0; m < kModes; ++m) p.state[mine + c * kModes + m] = state[c][m];
    }
  } else {
    float *const out = p.scratch + seg * per_segment + mine;
#pragma unroll
    for (int c = 0; c < kC; ++c)
#pragma unroll
      for (int m = 0; m < kModes; ++m) out[c * kModes + m] = state[c][m];
  }
}

// Segment length of the one-wave grid for `rows` rows: as many segments as the
// output pass has resident CTAs, none shorter than 64 rows, no more than the
// scratch holds.
// Eight rows of loads in flight per thread: with four the kernels waited on
// memory (12 KB in flight per SM), twelve cost the projection-fed form registers.
constexpr int kStreamUnroll = 8;

template <int kModes, bool kProj, int kC>
int stream_segments(const int rows, const int width, const std::size_t scratch_floats) {
  static const int resident = [] {
    int blocks = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(
            &blocks, modal_stream_kernel<kModes, kProj, true, kStreamUnroll, kC>, kStreamThreads, 0) != cudaSuccess ||
        blocks < 1)
      blocks = 1;
    return blocks;
  }();
  const int across = static_cast<int>(ceil_div_u(width / kC, kStreamThreads));
  int segments = std::max(1, kSmCount * resident / across);
  segments = std::min(segments, std::max(1, rows / 64));
  const std::size_t per_segment = static_cast<std::size_t>(width) * kModes;
  const std::size_t capacity = scratch_floats / per_segment;  // local states + the carried-in slot
  if (capacity < 2) return 1;
  return static_cast<int>(std::min<std::size_t>(segments, capacity - 1));
}

template <int kModes, bool kProj, int kC>
int launch_stream_form(ModalParams p, cudaStream_t stream) {
  const int rows = p.length - p.row_begin;
  const int segments = stream_segments<kModes, kProj, kC>(rows, p.width, p.scratch_floats);
  p.segment = (rows + segments - 1) / segments;
  p.segments = (rows + p.segment - 1) / p.segment;
  const unsigned int across = ceil_div_u(p.width / kC, kStreamThreads);
  if (p.segments > 1) {
    modal_stream_kernel<kModes, kProj, false, kStreamUnroll, kC>
        <<<dim3(across, p.segments - 1), kStreamThreads, 0, stream>>>(p);
    const int status = check_launch("modal segment-state kernel");
    if (status != kOk) return status;
  }
  modal_stream_kernel<kModes, kProj, true, kStreamUnroll, kC>
      <<<dim3(across, p.segments), kStreamThreads, 0, stream>>>(p);
  return check_launch("modal output kernel");
}

// One channel per thread where the registers of a pair cap the occupancy (16 modes: 96 of them
// hold poles, residues and states); pairs where they do not.
template <int kModes, bool kProj>
int launch_stream(const ModalParams &p, cudaStream_t stream) {
  static const bool pairs_only = [] {
    const char *const flag = std::getenv("EVO_B200_MODAL_PAIRS");
    return flag != nullptr && flag[0] == '1';
  }();
  if constexpr (kModes >= 8) {
    if (!pairs_only) return launch_stream_form<kModes, kProj, 1>(p, stream);
  }
  return launch_stream_form<kModes, kProj, 2>(p, stream);
}

template <int kModes>
int launch_modal(const ModalParams &p, const bool from_projection, cudaStream_t stream) {
  return from_projection ? launch_stream<kModes, true>(p, stream) : launch_stream<kModes, false>(p, stream);
}

}  // namespace

std::size_t modal_scratch_floats(const std::size_t length,
                                 const std::size_t width,
                                 const std::size_t modes) {
  if (length == 0 || width == 0) return 0;
  // One end state per segment of the one-wave grid (at most four resident CTAs
  // per SM, segments of at least 64 rows) and the carried-in slot.
  const std::size_t across = (width / 2 + kStreamThreads - 1) / kStreamThreads;
  const std::size_t segments =
      std::max<std::size_t>(1, std::min<std::size_t>(length / 64, static_cast<std::size_t>(kSmCount) * 4 / across));
  return (segments + 2) * width * modes;
}

// Any width and any state size up to 32 (the model shapes use even widths and 16 modes; upstream's
// operator tests use 7 x 3): a thread owns a channel and walks the rows in order, the modal state in
// registers.  Same rounding points as the chunked kernels: the first prefill rounds the convolution,
// the direct product and their sum to BF16 before the outer gate; a continuation rounds once.
namespace {
constexpr int kAnyModes = 32;

__global__ void __launch_bounds__(128)
modal_prefill_any_kernel(const bf16 *__restrict__ x2, const bf16 *__restrict__ x1, const bf16 *__restrict__ value,
                         const bf16 *__restrict__ direct, const float *__restrict__ log_poles,
                         const float *__restrict__ residues, float *__restrict__ state, bf16 *__restrict__ pregate,
                         bf16 *__restrict__ output, const int row_begin, const int length, const int width,
                         const int modes, const bool continue_from_state) {
  const int channel = blockIdx.x * blockDim.x + threadIdx.x;
  if (channel >= width) return;
  float pole[kAnyModes], residue[kAnyModes], held[kAnyModes];
  for (int m = 0; m < modes; ++m) {
    const std::size_t q = static_cast<std::size_t>(channel) * modes + m;
    pole[m] = expf(log_poles[q]);
    residue[m] = residues[q];
    held[m] = continue_from_state ? state[q] : 0.0F;
  }
  const float d = bf2f(direct[channel]);
  for (int t = row_begin; t < length; ++t) {
    const std::size_t at = static_cast<std::size_t>(t) * width + channel;
    const bf16 gated = f2bf(__fmul_rn(bf2f(x1[at]), bf2f(value[at])));
    if (pregate != nullptr) pregate[at] = gated;
    const float u = bf2f(gated);
    float modal = 0.0F;
    for (int m = 0; m < modes; ++m) {
      held[m] = fmaf(pole[m], held[m], u);
      modal = fmaf(residue[m], held[m], modal);
    }
    const float gate_value = bf2f(x2[at]);
    if (continue_from_state) {
      output[at] = f2bf(__fmul_rn(gate_value, fmaf(d, u, modal)));
    } else {
      const float mixed = rbf(__fadd_rn(rbf(modal), rbf(__fmul_rn(u, d))));
      output[at] = f2bf(__fmul_rn(mixed, gate_value));
    }
  }
  if (state != nullptr)
    for (int m = 0; m < modes; ++m) state[static_cast<std::size_t>(channel) * modes + m] = held[m];
}

bool takes_chunked_kernels(const ModalArgs &a) {
  return a.width % 2 == 0 && (a.modes == 1 || a.modes == 2 || a.modes == 4 || a.modes == 8 || a.modes == 16);
}

int modal_prefill_any(const ModalArgs &a, cudaStream_t stream) {
  if (a.projection != nullptr)
    return fail(kUnsupported, "modal prefill from the raw projection needs an even width and 1, 2, 4, 8 or 16 modes");
  if (a.x2 == nullptr || a.x1 == nullptr || a.value == nullptr || a.direct == nullptr || a.log_poles == nullptr ||
      a.residues == nullptr || a.output == nullptr || a.width == 0 || a.modes == 0)
    return fail(kInvalidArgument, "modal prefill arguments are invalid");
  if (a.modes > kAnyModes) return fail(kUnsupported, "modal state size must be at most 32");
  if (a.continue_from_state && a.state == nullptr) return fail(kInvalidArgument, "modal continuation needs a state");
  if (a.length > 0x7fffff00U || a.width > 0x3fffffffU || a.row_begin > a.length)
    return fail(kInvalidArgument, "modal prefill dimensions are too large");
  if (a.length == a.row_begin) return kOk;
  modal_prefill_any_kernel<<<ceil_div_u(a.width, 128), 128, 0, stream>>>(
      static_cast<const bf16 *>(a.x2), static_cast<const bf16 *>(a.x1), static_cast<const bf16 *>(a.value),
      static_cast<const bf16 *>(a.direct), a.log_poles, a.residues, a.state, static_cast<bf16 *>(a.pregate),
      static_cast<bf16 *>(a.output), static_cast<int>(a.row_begin), static_cast<int>(a.length),
      static_cast<int>(a.width), static_cast<int>(a.modes), a.continue_from_state);
  return check_launch("modal prefill kernel (any shape)");
}
}  // namespace

int modal_prefill(const ModalArgs &a, cudaStream_t stream) {
  if (a.width != 0 && a.modes != 0 && !takes_chunked_kernels(a)) return modal_prefill_any(a, stream);
  const bool from_projection = a.projection != nullptr;
  if (a.direct == nullptr || a.log_poles == nullptr || a.residues == nullptr ||
      a.output == nullptr || a.scratch == nullptr || a.width == 0 ||
      a.width % 2 != 0 || a.modes == 0)
    return fail(kInvalidArgument, "modal prefill arguments are invalid");
  if (from_projection
          ? (a.short_filter == nullptr || a.short_taps != 3)
          : (a.x2 == nullptr || a.x1 == nullptr || a.value == nullptr))
    return fail(kInvalidArgument, "modal prefill inputs are incomplete");
  if (a.continue_from_state && a.state == nullptr)
    return fail(kInvalidArgument, "modal continuation needs a state");
  if (a.length > 0x7fffff00U || a.width > 0x3fffffffU || a.row_begin > a.length)
    return fail(kInvalidArgument, "modal prefill dimensions are too large");
  if (a.length == a.row_begin) return kOk;
  ModalParams p{};
  p.x2 = static_cast<const bf16 *>(a.x2);
  p.x1 = static_cast<const bf16 *>(a.x1);
  p.value = static_cast<const bf16 *>(a.value);
  p.projection = static_cast<const bf16 *>(a.projection);
  p.short_filter = static_cast<const bf16 *>(a.short_filter);
  p.direct = static_cast<const bf16 *>(a.direct);
  p.log_poles = a.log_poles;
  p.residues = a.residues;
  p.output = static_cast<bf16 *>(a.output);
  p.pregate = static_cast<bf16 *>(a.pregate);
  p.state = a.state;
  p.scratch = a.scratch;
  p.length = static_cast<int>(a.length);
  p.width = static_cast<int>(a.width);
  p.row_begin = static_cast<int>(a.row_begin);
  p.pairs = static_cast<int>(a.width / 2);
  p.continue_from_state = a.continue_from_state;
  // sized by the rows of this call: a caller's buffer holds at least this much for any window of its length
  p.scratch_floats = modal_scratch_floats(a.length - a.row_begin, a.width, a.modes);
  p.short_cache = from_projection ? a.short_cache : nullptr;  // short_taps == 3 was checked above
  int status;
  switch (a.modes) {
    case 16: status = launch_modal<16>(p, from_projection, stream); break;
    case 8: status = launch_modal<8>(p, from_projection, stream); break;
    case 4: status = launch_modal<4>(p, from_projection, stream); break;
    case 2: status = launch_modal<2>(p, from_projection, stream); break;
    case 1: status = launch_modal<1>(p, from_projection, stream); break;
    default:
      return fail(kUnsupported, "modal state size must be 1, 2, 4, 8 or 16");
  }
  return status;
}

// ------------------------------------------------- allocation-free variant
// Segment-state scratch for callers that cannot allocate device memory: a
// fixed array that lives in the library image on every GPU that loads it.
constexpr std::size_t kStaticScratchFloats = std::size_t{4} << 20;  // 16 MiB
static __device__ __align__(256) float g_static_modal_scratch[kStaticScratchFloats];

namespace {
// Device address of the array above, looked up once per device.  The symbol
// name is only meaningful to the host as a handle; kernels need this address.
int static_scratch_address(float **out) {
  static std::mutex mutex;
  static float *addresses[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64)
    return fail(kCuda, "cannot query the current CUDA device");
  std::lock_guard<std::mutex> lock(mutex);
  if (addresses[device] == nullptr) {
    void *address = nullptr;
    const cudaError_t error = cudaGetSymbolAddress(&address, g_static_modal_scratch);
    if (error != cudaSuccess || address == nullptr)
      return fail(kCuda, std::string("cannot resolve the static modal scratch: ") +
                             cudaGetErrorString(error));
    addresses[device] = static_cast<float *>(address);
  }
  *out = addresses[device];
  return kOk;
}
}  // namespace

int modal_prefill_static_scratch(const ModalArgs &a, cudaStream_t stream) {
  if (a.width != 0 && a.modes != 0 && !takes_chunked_kernels(a)) return modal_prefill_any(a, stream);  // needs no scratch
  if (a.projection != nullptr || a.x2 == nullptr || a.x1 == nullptr || a.value == nullptr ||
      a.direct == nullptr || a.log_poles == nullptr || a.residues == nullptr ||
      a.output == nullptr || a.width == 0 || a.width % 2 != 0 || a.modes == 0)
    return fail(kInvalidArgument, "allocation-free modal prefill arguments are invalid");
  if (a.continue_from_state && a.state == nullptr)
    return fail(kInvalidArgument, "modal continuation needs a state");
  if (a.length > 0x7fffff00U || a.width > 0x3fffffffU)
    return fail(kInvalidArgument, "modal prefill dimensions are too large");
  if (a.length == 0) return kOk;
  const std::size_t per_segment = a.width * a.modes;
  if (per_segment > kStaticScratchFloats)
    return fail(kInvalidArgument,
                "allocation-free modal prefill: width*modes = " + std::to_string(per_segment) +
                    " floats per segment exceeds the fixed scratch of " +
                    std::to_string(kStaticScratchFloats) + " floats");
  float *scratch = nullptr;
  const int located = static_scratch_address(&scratch);
  if (located != kOk) return located;
  ModalParams p{};
  p.x2 = static_cast<const bf16 *>(a.x2);
  p.x1 = static_cast<const bf16 *>(a.x1);
  p.value = static_cast<const bf16 *>(a.value);
  p.direct = static_cast<const bf16 *>(a.direct);
  p.log_poles = a.log_poles;
  p.residues = a.residues;
  p.output = static_cast<bf16 *>(a.output);
  p.pregate = static_cast<bf16 *>(a.pregate);
  p.state = a.state;
  p.scratch = scratch;
  p.length = static_cast<int>(a.length);
  p.width = static_cast<int>(a.width);
  p.pairs = static_cast<int>(a.width / 2);
  p.continue_from_state = a.continue_from_state;
  p.scratch_floats = kStaticScratchFloats;  // fewer, longer segments when the array holds fewer states
  switch (a.modes) {
    case 16: return launch_modal<16>(p, false, stream);
    case 8: return launch_modal<8>(p, false, stream);
    case 4: return launch_modal<4>(p, false, stream);
    case 2: return launch_modal<2>(p, false, stream);
    case 1: return launch_modal<1>(p, false, stream);
    default: return fail(kUnsupported, "modal state size must be 1, 2, 4, 8 or 16");
  }
}

int modal_decode(const void *x2, const void *x1, const void *value,
                 const void *direct, const float *log_poles,
                 const float *residues, const std::size_t width,
                 const std::size_t modes, float *state, void *pregate,
                 void *output, cudaStream_t stream) {
  if (x2 == nullptr || x1 == nullptr || value == nullptr || direct == nullptr ||
      log_poles == nullptr || residues == nullptr || state == nullptr ||
      output == nullptr || width == 0 || modes == 0 || modes > 32)
    return fail(kInvalidArgument, "modal decode arguments are invalid");
  if (width > 0x3ffffffU) return fail(kInvalidArgument, "modal decode is too wide");
  modal_decode_warp_kernel<<<ceil_div_u(width * 32, kDecodeThreads), kDecodeThreads, 0, stream>>>(
      static_cast<const bf16 *>(x2), static_cast<const bf16 *>(x1),
      static_cast<const bf16 *>(value), static_cast<const bf16 *>(direct),
      log_poles, residues, state, static_cast<bf16 *>(pregate),
      static_cast<bf16 *>(output), static_cast<int>(width),
      static_cast<int>(modes));
  return check_launch("modal decode kernel");
}

int modal_taps(const void *gated, const float *log_poles, const float *residues, const std::size_t length,
               const std::size_t width, const std::size_t modes, float *filter, float *convolution,
               cudaStream_t stream) {
  if (log_poles == nullptr || residues == nullptr || (filter == nullptr && convolution == nullptr) ||
      (convolution != nullptr && gated == nullptr) || width == 0 || modes == 0 || modes > 32 ||
      length > 0x7fffffffU || width > 0x7fffffffU)
    return fail(kInvalidArgument, "modal tap arguments are invalid");
  if (length == 0) return kOk;
  modal_taps_kernel<<<ceil_div_u(width, 64), 64, 0, stream>>>(static_cast<const bf16 *>(gated), log_poles, residues,
                                                              filter, convolution, static_cast<int>(length),
                                                              static_cast<int>(width), static_cast<int>(modes));
  return check_launch("modal tap kernel");
}

}  // namespace evob
