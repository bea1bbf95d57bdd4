// One cached-decode step of a Hyena mixer in one launch.
//
// For a single new token the unfused path runs, per block, the 3-tap
// featurizer step over the [3 width] projection and its cache advance, the
// (x2, x1, v) split, the x1*v gate, the inner FIR step (or the modal step) with
// its cache update, and the x2 post-gate: four to seven launches that each move
// a few KB.  Here a warp owns one channel and does all of it:
//   lanes 0..2   featurizer step of the channel's three projection columns
//                (two cached rows + the new one), cache shifted in place;
//   all lanes    the inner FIR history (lane L owns entries L, 32+L, ...) or
//                the modal state (lane m owns mode m), folded with the same
//                32-slot trees as the unfused kernels, history shifted in place;
//   lane 0       direct term, post-gate, store.
// Every product, sum and rounding is the one the unfused kernels make, in the
// same order (upstream pins them: src/cuda/hyena.cu:275-416 for the FIR steps,
// :718-761 for the modal step), so the results are bit-identical.  Histories
// must be full (position >= taps - 1); shorter histories take the unfused path.
#include "common.cuh"
#include "ops_internal.hpp"

namespace evob {
namespace {

constexpr int kThreads = 256;

struct Params {
  const bf16 *projection, *short_filter, *direct;
  const void *filter;
  const float *log_poles, *residues;
  float *short_cache, *inner_cache, *modal_state;
  bf16 *output;
  int width, channels_per_group, taps, modes;
  bool filter_is_f32, cross_correlation;
};

__device__ __forceinline__ float filter_tap(const void *filter, const bool is_f32, const std::size_t index) {
  return is_f32 ? static_cast<const float *>(filter)[index] : bf2f(static_cast<const bf16 *>(filter)[index]);
}

template <bool kModal>
__global__ void __launch_bounds__(kThreads)
mixer_decode_kernel(const Params p) {
  // lets a one-row projection launched with programmatic stream serialisation start (and fetch its
  // weights) under this kernel; it still waits for this grid to finish before it reads the result
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int channel = (blockIdx.x * kThreads + threadIdx.x) / 32;
  const int lane = threadIdx.x % 32;
  if (channel >= p.width) return;

  // featurizer step: 3 taps, cross-correlation (oldest cached row meets tap 0)
  float z = 0.0F;
  if (lane < 3) {
    const std::size_t column = static_cast<std::size_t>(channel) * 3 + lane;
    float *const row = p.short_cache + column * 2;
    const float older = row[0], newer = row[1];
    const bf16 *const w = p.short_filter + column * 3;
    // slots 0 and 1 of the 32-slot tree; the other slots are +0 and only matter for the sign of zero
    const float t0 = __fadd_rn(0.0F, __fmul_rn(older, bf2f(w[0])));
    const float t1 = __fadd_rn(0.0F, __fmul_rn(newer, bf2f(w[1])));
    const float current = bf2f(p.projection[column]);
    z = rbf(__fadd_rn(__fmul_rn(current, bf2f(w[2])), __fadd_rn(t0, t1)));
    row[0] = newer;
    row[1] = current;
  }
  const float x2 = __shfl_sync(0xffffffffU, z, 0);
  const float x1 = __shfl_sync(0xffffffffU, z, 1);
  const float v = __shfl_sync(0xffffffffU, z, 2);
  const float gated = rbf(x1 * v);

  if constexpr (kModal) {
    float term = 0.0F;
    if (lane < p.modes) {
      const std::size_t q = static_cast<std::size_t>(channel) * p.modes + lane;
      const float updated = __fadd_rn(__fmul_rn(expf(p.log_poles[q]), p.modal_state[q]), gated);
      p.modal_state[q] = updated;
      term = __fmul_rn(p.residues[q], updated);
    }
#pragma unroll
    for (int offset = 16; offset != 0; offset /= 2) {
      const float other = __shfl_down_sync(0xffffffffU, term, offset);
      if (lane < 32 - offset) term = __fadd_rn(term, other);
    }
    if (lane == 0) {
      const float direct_product = rbf(bf2f(p.direct[channel]) * gated);
      p.output[channel] = f2bf(__fmul_rn(x2, __fadd_rn(term, direct_product)));
    }
  } else {
    const int cache_size = p.taps - 1;
    const std::size_t group = channel / p.channels_per_group;
    float *const row = p.inner_cache + static_cast<std::size_t>(channel) * cache_size;
    float history[4];  // taps <= 128
    float term = 0.0F;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int a = 32 * k + lane;
      history[k] = a < cache_size ? row[a] : 0.0F;
      if (a < cache_size) {
        const int tap = p.cross_correlation ? a : cache_size - a;
        term = __fadd_rn(term, __fmul_rn(history[k], filter_tap(p.filter, p.filter_is_f32, group * p.taps + tap)));
      }
    }
#pragma unroll
    for (int offset = 16; offset != 0; offset /= 2) {
      const float other = __shfl_down_sync(0xffffffffU, term, offset);
      if (lane < offset) term = __fadd_rn(term, other);
    }
    __syncwarp();  // every lane has read its entries before any is overwritten
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int a = 32 * k + lane;
      if (a >= 1 && a < cache_size) row[a - 1] = history[k];
    }
    if (lane == 0) {
      row[cache_size - 1] = gated;
      const int current_tap = p.cross_correlation ? cache_size : 0;
      float total =
          __fadd_rn(__fmul_rn(gated, filter_tap(p.filter, p.filter_is_f32, group * p.taps + current_tap)), term);
      if (p.direct != nullptr) total = __fadd_rn(total, __fmul_rn(bf2f(p.direct[channel]), gated));
      p.output[channel] = f2bf(rbf(total) * x2);
    }
  }
}

}  // namespace

int hyena_decode_mixer(const DecodeMixerArgs &a, cudaStream_t stream) {
  const bool modal = a.log_poles != nullptr;
  if (a.projection == nullptr || a.short_filter == nullptr || a.short_cache == nullptr || a.output == nullptr ||
      a.width == 0 || a.width > 0x3ffffffU)
    return fail(kInvalidArgument, "decode mixer arguments are invalid");
  if (modal ? (a.residues == nullptr || a.modal_state == nullptr || a.direct == nullptr || a.modes == 0 ||
               a.modes > 32)
            : (a.filter == nullptr || a.inner_cache == nullptr || a.groups == 0 || a.width % a.groups != 0 ||
               a.taps < 2 || a.taps > 128))
    return fail(kInvalidArgument, "decode mixer operator arguments are invalid");
  Params p{};
  p.projection = static_cast<const bf16 *>(a.projection);
  p.short_filter = static_cast<const bf16 *>(a.short_filter);
  p.direct = static_cast<const bf16 *>(a.direct);
  p.filter = a.filter;
  p.log_poles = a.log_poles;
  p.residues = a.residues;
  p.short_cache = a.short_cache;
  p.inner_cache = a.inner_cache;
  p.modal_state = a.modal_state;
  p.output = static_cast<bf16 *>(a.output);
  p.width = static_cast<int>(a.width);
  p.channels_per_group = modal ? 1 : static_cast<int>(a.width / a.groups);
  p.taps = static_cast<int>(a.taps);
  p.modes = static_cast<int>(a.modes);
  p.filter_is_f32 = a.filter_is_f32;
  p.cross_correlation = a.cross_correlation;
  const unsigned int grid = ceil_div_u(a.width * 32, kThreads);
  if (modal)
    mixer_decode_kernel<true><<<grid, kThreads, 0, stream>>>(p);
  else
    mixer_decode_kernel<false><<<grid, kThreads, 0, stream>>>(p);
  return check_launch("decode mixer kernel");
}

}  // namespace evob
