// Short (k=3), short-explicit (HCS, k=7) and medium-regularised (HCM, k=128)
// causal depthwise FIR operators of the Hyena mixers.
//
// gated_fir_prefill is the fused prefill operator: one pass reads either the
// three gate tensors x2/x1/v or the raw interleaved projection (applying the
// 3-tap featurizer filter on the fly), forms u = bf16(x1*v), convolves it with
// the grouped inner filter out of a shared-memory time tile, adds the direct
// term, rounds, applies the x2 post-gate and writes the mixer output - the
// work upstream spreads over a short-FIR pass, a split pass, two gate passes
// and a direct or FFT convolution (src/cuda/hyena.cu:243-272, 418-519,
// 1792-1992; src/cuda/model.cu:1431-1520).  Rounding points are kept:
// bf16 after the featurizer FIR, after x1*v, after the inner FIR (+direct), and
// after the post-gate.  Taps are accumulated oldest-input-first with FMA, the
// order of upstream's direct kernel.
//
// fir_prefill / fir_step are the unfused operators (sliding register window
// per channel; warp per output with upstream's pinned decode/continue
// reduction tree as a shuffle fold, src/cuda/hyena.cu:275-416).
#include "common.cuh"
#include "ops_internal.hpp"

namespace evob {
namespace {

constexpr int kThreads = 256;
constexpr int kTileT = 128;       // outputs per CTA along time
constexpr int kTilePairs = 32;    // channel pairs per CTA (64 channels)
constexpr int kRun = 16;          // consecutive outputs per thread
constexpr int kMaxTaps = 128;

__device__ __forceinline__ float load_filter(const void *filter,
                                             const bool is_f32,
                                             const std::size_t index) {
  return is_f32 ? static_cast<const float *>(filter)[index]
                : bf2f(static_cast<const bf16 *>(filter)[index]);
}

struct FusedParams {
  const bf16 *x2, *x1, *value;
  const bf16 *projection;
  const bf16 *short_filter;
  const void *filter;
  const bf16 *direct;
  bf16 *output;
  bf16 *pregate;
  float *inner_cache;
  int length, row_begin, width, taps, padded_taps, channels_per_group;
  bool filter_is_f32, cross_correlation;
};

// 3-tap featurizer over one projection stream pair; rows before the sequence
// start read as zero, which leaves the FMA chain bit-identical to skipping them.
__device__ __forceinline__ void short_fir_pair(
    const bf16 *projection, const int width3, const int t, const int stream,
    const float (&w)[2][3], float &out0, float &out1) {
  float a0 = 0.0F, a1 = 0.0F;
#pragma unroll
  for (int j = 0; j < 3; ++j) {
    const int row = t - (2 - j);
    if (row >= 0) {
      const std::size_t base = static_cast<std::size_t>(row) * width3 + stream;
      a0 = fmaf(bf2f(projection[base]), w[0][j], a0);
      a1 = fmaf(bf2f(projection[base + 3]), w[1][j], a1);
    }
  }
  out0 = rbf(a0);
  out1 = rbf(a1);
}

template <bool kFromProjection>
__global__ void __launch_bounds__(kThreads)
gated_fir_kernel(const FusedParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int halo = p.padded_taps - 1;
  // u tile: [(kTileT + halo)][kTilePairs] packed bf16x2
  std::uint32_t *const u_tile = reinterpret_cast<std::uint32_t *>(smem_raw);
  // x2 tile: [kTileT][kTilePairs] packed bf16x2
  std::uint32_t *const x2_tile = u_tile + (kTileT + halo) * kTilePairs;
  // filter: [padded_taps][kTilePairs] float2, indexed by delay
  float2 *const h_tile =
      reinterpret_cast<float2 *>(x2_tile + kTileT * kTilePairs);

  const int t0 = p.row_begin + blockIdx.x * kTileT;
  const int pair0 = blockIdx.y * kTilePairs;
  const int lane_pair = threadIdx.x % kTilePairs;
  const int sub = threadIdx.x / kTilePairs;  // 0..7
  const int c0 = (pair0 + lane_pair) * 2;
  const bool channel_ok = c0 < p.width;
  const int width3 = p.width * 3;

  // ---- filter -> shared, indexed by delay (input age)
  for (int d = sub; d < p.padded_taps; d += kThreads / kTilePairs) {
    float2 h = make_float2(0.0F, 0.0F);
    if (channel_ok && d < p.taps) {
      const int tap = p.cross_correlation ? p.taps - 1 - d : d;
      h.x = load_filter(p.filter, p.filter_is_f32,
                        static_cast<std::size_t>(c0 / p.channels_per_group) *
                                p.taps + tap);
      h.y = load_filter(p.filter, p.filter_is_f32,
                        static_cast<std::size_t>((c0 + 1) / p.channels_per_group) *
                                p.taps + tap);
    }
    h_tile[d * kTilePairs + lane_pair] = h;
  }

  // ---- u (and x2) tiles
  float sw[3][2][3];  // [stream x2/x1/v][channel of the pair][tap]
  if constexpr (kFromProjection) {
    if (channel_ok) {
#pragma unroll
      for (int s = 0; s < 3; ++s)
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int j = 0; j < 3; ++j)
            sw[s][c][j] = bf2f(
                p.short_filter[(static_cast<std::size_t>(c0 + c) * 3 + s) * 3 + j]);
    }
  }
  const int real_halo = p.taps - 1;
  for (int r = sub; r < kTileT + halo; r += kThreads / kTilePairs) {
    const int t = t0 - halo + r;
    std::uint32_t packed_u = 0U;
    if (channel_ok && t >= 0 && t < p.length && t >= t0 - real_halo) {
      float u0, u1;
      if constexpr (kFromProjection) {
        float a0, a1, b0, b1;
        short_fir_pair(p.projection, width3, t, c0 * 3 + 1, sw[1], a0, a1);
        short_fir_pair(p.projection, width3, t, c0 * 3 + 2, sw[2], b0, b1);
        u0 = rbf(a0 * b0);
        u1 = rbf(a1 * b1);
      } else {
        const std::size_t index = static_cast<std::size_t>(t) * p.width + c0;
        const std::uint32_t a = *reinterpret_cast<const std::uint32_t *>(p.x1 + index);
        const std::uint32_t b = *reinterpret_cast<const std::uint32_t *>(p.value + index);
        u0 = rbf(__uint_as_float(a << 16U) * __uint_as_float(b << 16U));
        u1 = rbf(__uint_as_float(a & 0xffff0000U) * __uint_as_float(b & 0xffff0000U));
      }
      packed_u = (__float_as_uint(u0) >> 16U) | (__float_as_uint(u1) & 0xffff0000U);
      if (t >= t0) {
        const std::size_t index = static_cast<std::size_t>(t) * p.width + c0;
        if (p.pregate != nullptr)
          *reinterpret_cast<std::uint32_t *>(p.pregate + index) = packed_u;
        if (p.inner_cache != nullptr && real_halo > 0) {
          const int slot = t - (p.length - real_halo);
          if (slot >= 0) {
            p.inner_cache[static_cast<std::size_t>(c0) * real_halo + slot] = u0;
            p.inner_cache[static_cast<std::size_t>(c0 + 1) * real_halo + slot] = u1;
          }
        }
      }
    }
    u_tile[r * kTilePairs + lane_pair] = packed_u;
    if (r >= halo) {
      std::uint32_t packed_x2 = 0U;
      if (channel_ok && t < p.length) {
        if constexpr (kFromProjection) {
          float z0, z1;
          short_fir_pair(p.projection, width3, t, c0 * 3, sw[0], z0, z1);
          packed_x2 = (__float_as_uint(z0) >> 16U) | (__float_as_uint(z1) & 0xffff0000U);
        } else {
          packed_x2 = *reinterpret_cast<const std::uint32_t *>(
              p.x2 + static_cast<std::size_t>(t) * p.width + c0);
        }
      }
      x2_tile[(r - halo) * kTilePairs + lane_pair] = packed_x2;
    }
  }
  __syncthreads();

  // ---- convolution: thread owns kRun consecutive outputs of one pair
  const int run0 = sub * kRun;  // first output row of this thread in the tile
  float acc0[kRun], acc1[kRun];
#pragma unroll
  for (int r = 0; r < kRun; ++r) acc0[r] = acc1[r] = 0.0F;
  for (int d0 = p.padded_taps - kRun; d0 >= 0; d0 -= kRun) {
    // window rows: output r with delay d reads tile row halo + run0 + r - d.
    // For d in [d0, d0+kRun) and r in [0,kRun): offsets from
    // base = halo + run0 - d0 - (kRun-1) span 0 .. 2*kRun-2.
    const int base = halo + run0 - d0 - (kRun - 1);
    float w0[2 * kRun - 1], w1[2 * kRun - 1];
#pragma unroll
    for (int i = 0; i < 2 * kRun - 1; ++i) {
      const std::uint32_t packed = u_tile[(base + i) * kTilePairs + lane_pair];
      w0[i] = __uint_as_float(packed << 16U);
      w1[i] = __uint_as_float(packed & 0xffff0000U);
    }
#pragma unroll
    for (int dd = kRun - 1; dd >= 0; --dd) {  // oldest input first
      const float2 h = h_tile[(d0 + dd) * kTilePairs + lane_pair];
#pragma unroll
      for (int r = 0; r < kRun; ++r) {
        // row offset = r - dd + (kRun-1)
        acc0[r] = fmaf(w0[r - dd + kRun - 1], h.x, acc0[r]);
        acc1[r] = fmaf(w1[r - dd + kRun - 1], h.y, acc1[r]);
      }
    }
  }
  if (!channel_ok) return;
  float direct0 = 0.0F, direct1 = 0.0F;
  if (p.direct != nullptr) {
    direct0 = bf2f(p.direct[c0]);
    direct1 = bf2f(p.direct[c0 + 1]);
  }
#pragma unroll
  for (int r = 0; r < kRun; ++r) {
    const int t = t0 + run0 + r;
    if (t >= p.length) break;
    float y0 = acc0[r], y1 = acc1[r];
    if (p.direct != nullptr) {
      const std::uint32_t packed = u_tile[(halo + run0 + r) * kTilePairs + lane_pair];
      y0 = fmaf(direct0, __uint_as_float(packed << 16U), y0);
      y1 = fmaf(direct1, __uint_as_float(packed & 0xffff0000U), y1);
    }
    const std::uint32_t gate = x2_tile[(run0 + r) * kTilePairs + lane_pair];
    const float o0 = rbf(y0) * __uint_as_float(gate << 16U);
    const float o1 = rbf(y1) * __uint_as_float(gate & 0xffff0000U);
    *reinterpret_cast<std::uint32_t *>(
        p.output + static_cast<std::size_t>(t) * p.width + c0) = pack_bf16x2(o0, o1);
  }
}

// -------------------------------------------------------------- unfused
// History cache of a depthwise FIR: per channel the last cache_size inputs in
// chronological order, left-padded with zeros.  A warp owns a channel, reads
// the row it is about to shift into registers (lane L holds slots L, 32+L, ...),
// and writes slot s from slot s+length of the old row or, past its end, from
// the new rows - so a fill after a prefill (`fresh`: the old row counts as
// zeros) and an advance after a continuation chunk are the same kernel.
constexpr int kHistorySlotsPerLane = 8;  // cache_size <= 256

__global__ void __launch_bounds__(kThreads)
history_update_kernel(const bf16 *__restrict__ input, float *__restrict__ cache, const int length,
                      const int channels, const int cache_size, const bool fresh) {
  const int channel = (blockIdx.x * kThreads + threadIdx.x) / 32;
  const int lane = threadIdx.x % 32;
  if (channel >= channels) return;
  float *const row = cache + static_cast<std::size_t>(channel) * cache_size;
  float moved[kHistorySlotsPerLane];
#pragma unroll
  for (int k = 0; k < kHistorySlotsPerLane; ++k) {
    const int slot = 32 * k + lane;
    const long source = static_cast<long>(slot) + length;
    moved[k] = 0.0F;
    if (slot >= cache_size) continue;
    if (source < cache_size) {
      if (!fresh) moved[k] = row[source];
    } else {
      moved[k] = bf2f(input[static_cast<std::size_t>(source - cache_size) * channels + channel]);
    }
  }
  __syncwarp();  // all old slots are in registers before any is overwritten
#pragma unroll
  for (int k = 0; k < kHistorySlotsPerLane; ++k) {
    const int slot = 32 * k + lane;
    if (slot < cache_size) row[slot] = moved[k];
  }
}

// Unfused prefill FIR.  A thread owns one channel and a run of kRows
// consecutive outputs; the taps are the outer loop, and the kRows inputs that
// meet tap j are a register window that slides by one row from tap to tap (one
// new load per tap instead of kRows).  Each output still accumulates its taps
// in index order 0..taps-1 with one FMA per tap and skips the taps that reach
// before the sequence start, which is the summation upstream's direct kernel
// defines (src/cuda/hyena.cu:243-272).
constexpr int kRows = 8;

template <bool kCross>
__global__ void __launch_bounds__(kThreads)
fir_run_kernel(const bf16 *__restrict__ input, const void *__restrict__ filter, const bool filter_is_f32,
               const bf16 *__restrict__ bias, const bool multiply_bias, bf16 *__restrict__ output,
               const std::size_t length, const std::size_t channels, const std::size_t channels_per_group,
               const int taps) {
  const std::size_t runs = (length + kRows - 1) / kRows;
  const std::size_t item = static_cast<std::size_t>(blockIdx.x) * kThreads + threadIdx.x;
  if (item >= runs * channels) return;
  const std::size_t channel = item % channels;
  const long first = static_cast<long>(item / channels) * kRows;
  const std::size_t group = channel / channels_per_group;
  const auto sample = [&](const long row) -> float {
    return row >= 0 && row < static_cast<long>(length) ? bf2f(input[static_cast<std::size_t>(row) * channels + channel])
                                                       : 0.0F;
  };
  // delay of tap j: taps-1-j (cross-correlation) or j (convolution)
  int delay = kCross ? taps - 1 : 0;
  float window[kRows], total[kRows];
#pragma unroll
  for (int r = 0; r < kRows; ++r) {
    window[r] = sample(first + r - delay);
    total[r] = 0.0F;
  }
  for (int tap = 0; tap < taps; ++tap) {
    const float weight = load_filter(filter, filter_is_f32, group * taps + tap);
#pragma unroll
    for (int r = 0; r < kRows; ++r)
      if (first + r >= delay) total[r] = fmaf(window[r], weight, total[r]);
    if (tap + 1 == taps) break;
    if constexpr (kCross) {
      --delay;
#pragma unroll
      for (int r = 0; r + 1 < kRows; ++r) window[r] = window[r + 1];
      window[kRows - 1] = sample(first + kRows - 1 - delay);
    } else {
      ++delay;
#pragma unroll
      for (int r = kRows - 1; r > 0; --r) window[r] = window[r - 1];
      window[0] = sample(first - delay);
    }
  }
#pragma unroll
  for (int r = 0; r < kRows; ++r) {
    const long row = first + r;
    if (row >= static_cast<long>(length)) break;
    const std::size_t at = static_cast<std::size_t>(row) * channels + channel;
    float value = total[r];
    if (bias != nullptr) {
      const float b = bf2f(bias[channel]);
      value = multiply_bias ? fmaf(b, bf2f(input[at]), value) : value + b;
    }
    output[at] = f2bf(value);
  }
}

// Continuation rows against the F32 history cache with the reduction upstream
// pins for its cached FIR (src/cuda/hyena.cu:275-330): every product rounded by
// itself, history entry a added into slot a % 32 in ascending a, the 32 slots
// folded 16/8/4/2/1, then the current sample's product, then the bias term.  A
// warp owns one (row, channel) output and a lane is a slot, so the slots are
// the lanes' private sums and the fold is five shuffles.  History entries come
// from the cache while they predate this chunk and from the chunk's own earlier
// rows after that.
__global__ void __launch_bounds__(kThreads)
fir_rows_warp_kernel(const bf16 *__restrict__ input, const void *__restrict__ filter, const bool filter_is_f32,
                     const bf16 *__restrict__ bias, const bool multiply_bias, const float *__restrict__ cache,
                     bf16 *__restrict__ output, const std::size_t length, const std::size_t channels,
                     const std::size_t channels_per_group, const int taps, const int cached,
                     const bool cross_correlation) {
  const std::size_t item = (static_cast<std::size_t>(blockIdx.x) * kThreads + threadIdx.x) / 32;
  const int lane = threadIdx.x % 32;
  if (item >= length * channels) return;
  const std::size_t channel = item % channels;
  const long row = static_cast<long>(item / channels);
  const std::size_t group = channel / channels_per_group;
  const int cache_size = taps - 1;
  const long seen = cached + row;                       // inputs before this row
  const int active = static_cast<int>(seen < cache_size ? seen : cache_size);
  const long oldest = seen - active;                    // index of history entry 0 among the seen inputs
  float slot = 0.0F;
  for (int a = lane; a < active; a += 32) {
    const long index = oldest + a;
    const float source = index < cached
                             ? cache[channel * cache_size + (cache_size - cached) + index]
                             : bf2f(input[static_cast<std::size_t>(index - cached) * channels + channel]);
    const int tap = cross_correlation ? a : active - a;
    slot = __fadd_rn(slot, __fmul_rn(source, load_filter(filter, filter_is_f32, group * taps + tap)));
  }
#pragma unroll
  for (int offset = 16; offset != 0; offset /= 2) {
    const float other = __shfl_down_sync(0xffffffffU, slot, offset);
    if (lane < offset) slot = __fadd_rn(slot, other);
  }
  if (lane != 0) return;
  const float current = bf2f(input[item]);
  const int current_tap = cross_correlation ? active : 0;
  float total = __fadd_rn(__fmul_rn(current, load_filter(filter, filter_is_f32, group * taps + current_tap)), slot);
  if (bias != nullptr) {
    const float b = bf2f(bias[channel]);
    total = __fadd_rn(total, multiply_bias ? __fmul_rn(b, current) : b);
  }
  output[item] = f2bf(total);
}

// Single-step form (cached decode) for long filters with a full history: one
// warp per channel.  Lane L owns history entries L, 32+L, 64+L, ... - exactly
// the slots of fir_rows_warp_kernel - and the 32-slot tree is folded with
// shuffles in the same order, so the result is bit-identical; the history row
// is read once, coalesced, and written back shifted by one with the new sample
// appended, which replaces the separate cache-advance launch.
__global__ void __launch_bounds__(kThreads)
fir_decode_warp_kernel(const bf16 *__restrict__ input, const void *__restrict__ filter,
                       const bool filter_is_f32, const bf16 *__restrict__ bias,
                       const bool multiply_bias, float *__restrict__ cache, bf16 *__restrict__ output,
                       const int channels, const int channels_per_group, const int taps,
                       const bool cross_correlation) {
  const int channel = (blockIdx.x * kThreads + threadIdx.x) / 32;
  const int lane = threadIdx.x % 32;
  if (channel >= channels) return;
  const int cache_size = taps - 1;
  const std::size_t group = channel / channels_per_group;
  float *const row = cache + static_cast<std::size_t>(channel) * cache_size;
  float history[4];  // taps <= 128
  float term = 0.0F;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int a = 32 * k + lane;
    history[k] = a < cache_size ? row[a] : 0.0F;
    if (a < cache_size) {
      const int tap = cross_correlation ? a : cache_size - a;
      term = __fadd_rn(term, __fmul_rn(history[k], load_filter(filter, filter_is_f32, group * taps + tap)));
    }
  }
#pragma unroll
  for (int offset = 16; offset != 0; offset /= 2) {
    const float other = __shfl_down_sync(0xffffffffU, term, offset);
    if (lane < offset) term = __fadd_rn(term, other);
  }
  const float current = bf2f(input[channel]);
  __syncwarp();  // every lane has read its entries before any is overwritten
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int a = 32 * k + lane;
    if (a >= 1 && a < cache_size) row[a - 1] = history[k];
  }
  if (lane == 0) {
    row[cache_size - 1] = current;
    const int current_tap = cross_correlation ? cache_size : 0;
    float total = __fadd_rn(
        __fmul_rn(current, load_filter(filter, filter_is_f32, group * taps + current_tap)), term);
    if (bias != nullptr) {
      const float b = bf2f(bias[channel]);
      total = __fadd_rn(total, multiply_bias ? __fmul_rn(b, current) : b);
    }
    output[channel] = f2bf(total);
  }
}

}  // namespace

// Odd widths (no model shape has one; upstream's operator tests do): the fused kernels work on channel
// pairs, so the operator runs as its three steps - inner gate into `pregate`, the plain FIR with the
// direct term as a multiply-input bias, outer gate in place - with the same BF16 rounding points.
static int gated_fir_prefill_unfused(const GatedFirArgs &a, cudaStream_t stream) {
  if (a.projection != nullptr || a.row_begin != 0)
    return fail(kUnsupported, "gated FIR at an odd width takes separate x2 / x1 / value inputs and whole sequences");
  if (a.pregate == nullptr)
    return fail(kInvalidArgument, "gated FIR at an odd width needs the pregate buffer for the inner gate");
  if (a.x2 == nullptr || a.x1 == nullptr || a.value == nullptr)
    return fail(kInvalidArgument, "gated FIR inputs are incomplete");
  if (a.length == 0) return kOk;
  const std::size_t elements = a.length * a.width;
  int status = gate(a.x1, a.value, a.pregate, elements, false, stream);
  if (status != kOk) return status;
  status = fir_prefill(a.pregate, a.filter, a.filter_is_f32, a.direct, a.direct != nullptr, a.length, a.width,
                       a.groups, a.taps, a.cross_correlation, a.output, a.inner_cache, stream);
  if (status != kOk) return status;
  return gate(a.output, a.x2, a.output, elements, false, stream);
}

int gated_fir_prefill_generic(const GatedFirArgs &a, cudaStream_t stream) {
  const bool from_projection = a.projection != nullptr;
  if (a.filter != nullptr && a.output != nullptr && a.width % 2 != 0 && a.groups != 0 && a.taps != 0 &&
      a.taps <= kMaxTaps && a.width % a.groups == 0)
    return gated_fir_prefill_unfused(a, stream);
  if (a.filter == nullptr || a.output == nullptr || a.width == 0 ||
      a.groups == 0 || a.taps == 0 || a.taps > kMaxTaps ||
      a.width % a.groups != 0 || a.width % 2 != 0)
    return fail(kInvalidArgument, "gated FIR arguments are invalid");
  if (from_projection
          ? (a.short_filter == nullptr || a.short_taps != 3)
          : (a.x2 == nullptr || a.x1 == nullptr || a.value == nullptr))
    return fail(kInvalidArgument, "gated FIR inputs are incomplete");
  if (a.length > 0x7fffff00U)
    return fail(kInvalidArgument, "gated FIR sequence is too long");
  if (a.inner_cache != nullptr && a.taps > 1) {
    if (cudaMemsetAsync(a.inner_cache, 0, a.width * (a.taps - 1) * sizeof(float),
                        stream) != cudaSuccess)
      return fail(kCuda, "cannot clear the FIR cache");
  }
  if (a.row_begin > a.length) return fail(kInvalidArgument, "gated FIR row window is invalid");
  if (a.length == a.row_begin) return kOk;
  FusedParams p{};
  p.row_begin = static_cast<int>(a.row_begin);
  p.x2 = static_cast<const bf16 *>(a.x2);
  p.x1 = static_cast<const bf16 *>(a.x1);
  p.value = static_cast<const bf16 *>(a.value);
  p.projection = static_cast<const bf16 *>(a.projection);
  p.short_filter = static_cast<const bf16 *>(a.short_filter);
  p.filter = a.filter;
  p.direct = static_cast<const bf16 *>(a.direct);
  p.output = static_cast<bf16 *>(a.output);
  p.pregate = static_cast<bf16 *>(a.pregate);
  p.inner_cache = a.inner_cache;
  p.length = static_cast<int>(a.length);
  p.width = static_cast<int>(a.width);
  p.taps = static_cast<int>(a.taps);
  p.padded_taps = static_cast<int>((a.taps + kRun - 1) / kRun * kRun);
  p.channels_per_group = static_cast<int>(a.width / a.groups);
  p.filter_is_f32 = a.filter_is_f32;
  p.cross_correlation = a.cross_correlation;
  const int halo = p.padded_taps - 1;
  const std::size_t smem = static_cast<std::size_t>(kTileT + halo) * kTilePairs * 4 +
                           static_cast<std::size_t>(kTileT) * kTilePairs * 4 +
                           static_cast<std::size_t>(p.padded_taps) * kTilePairs * 8;
  const dim3 grid(ceil_div_u(a.length - a.row_begin, kTileT), ceil_div_u(a.width / 2, kTilePairs));
  if (grid.y > 65535) return fail(kInvalidArgument, "gated FIR is too wide");
  auto *const kernel = from_projection ? gated_fir_kernel<true> : gated_fir_kernel<false>;
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(smem)) != cudaSuccess)
    return fail(kCuda, "cannot raise the gated FIR shared-memory limit");
  kernel<<<grid, kThreads, smem, stream>>>(p);
  int status = check_launch("gated FIR kernel");
  if (status != kOk) return status;
  if (a.short_cache != nullptr && from_projection && a.short_taps > 1)
    status = fill_fir_cache(p.projection, a.short_cache, a.length, a.width * 3, a.short_taps - 1, stream);
  return status;
}

// fresh: the cache holds nothing yet (fill after a prefill); otherwise it is
// shifted by `length` and the new rows are appended.
static int update_history(const void *input, float *cache, const std::size_t length, const std::size_t channels,
                          const std::size_t cache_size, const bool fresh, cudaStream_t stream) {
  if (cache_size > 32 * kHistorySlotsPerLane || channels > 0x3ffffffU || length > 0x7fffff00U)
    return fail(kInvalidArgument, "FIR history is longer than 256 entries or the tensor is too large");
  history_update_kernel<<<ceil_div_u(channels * 32, kThreads), kThreads, 0, stream>>>(
      static_cast<const bf16 *>(input), cache, static_cast<int>(length), static_cast<int>(channels),
      static_cast<int>(cache_size), fresh);
  return check_launch("FIR history kernel");
}

int fill_fir_cache(const void *input, float *cache, const std::size_t length,
                   const std::size_t channels, const std::size_t cache_size,
                   cudaStream_t stream) {
  if (input == nullptr || cache == nullptr || channels == 0)
    return fail(kInvalidArgument, "FIR cache fill arguments are invalid");
  if (cache_size == 0) return kOk;
  return update_history(input, cache, length, channels, cache_size, true, stream);
}

int fir_prefill(const void *input, const void *filter, const bool filter_is_f32,
                const void *bias, const bool multiply_bias,
                const std::size_t length, const std::size_t channels,
                const std::size_t groups, const std::size_t taps,
                const bool cross_correlation, void *output, float *cache,
                cudaStream_t stream) {
  if (input == nullptr || filter == nullptr || output == nullptr ||
      channels == 0 || groups == 0 || taps == 0 || channels % groups != 0)
    return fail(kInvalidArgument, "FIR prefill arguments are invalid");
  if (taps > 0x7fffffffU) return fail(kInvalidArgument, "FIR prefill arguments are invalid");
  if (length != 0) {
    const std::size_t items = (length + kRows - 1) / kRows * channels;
    if ((items + kThreads - 1) / kThreads > 0x7fffffffU) return fail(kInvalidArgument, "FIR prefill is too large");
    auto *const kernel = cross_correlation ? fir_run_kernel<true> : fir_run_kernel<false>;
    kernel<<<ceil_div_u(items, kThreads), kThreads, 0, stream>>>(
        static_cast<const bf16 *>(input), filter, filter_is_f32, static_cast<const bf16 *>(bias), multiply_bias,
        static_cast<bf16 *>(output), length, channels, channels / groups, static_cast<int>(taps));
    const int status = check_launch("FIR prefill kernel");
    if (status != kOk) return status;
  }
  if (cache != nullptr && taps > 1) return update_history(input, cache, length, channels, taps - 1, true, stream);
  return kOk;
}

int fir_step(const void *input, const void *filter, const bool filter_is_f32,
             const void *bias, const bool multiply_bias,
             const std::size_t length, const std::size_t channels,
             const std::size_t groups, const std::size_t taps,
             const bool cross_correlation, float *cache,
             const std::size_t cache_length, void *output,
             cudaStream_t stream) {
  if (input == nullptr || filter == nullptr || output == nullptr ||
      cache == nullptr || channels == 0 || groups == 0 || taps < 2 ||
      channels % groups != 0 || cache_length > taps - 1 || length == 0)
    return fail(kInvalidArgument, "FIR step arguments are invalid");
  if (length == 1 && taps > 33 && taps <= 128 && cache_length == taps - 1 && channels <= 0x3fffffU) {
    fir_decode_warp_kernel<<<ceil_div_u(channels * 32, kThreads), kThreads, 0, stream>>>(
        static_cast<const bf16 *>(input), filter, filter_is_f32, static_cast<const bf16 *>(bias),
        multiply_bias, cache, static_cast<bf16 *>(output), static_cast<int>(channels),
        static_cast<int>(channels / groups), static_cast<int>(taps), cross_correlation);
    return check_launch("FIR decode kernel");
  }
  const std::size_t warps = length * channels;
  if (warps > 0x3ffffffU || taps > 0x7fffffffU) return fail(kInvalidArgument, "FIR step is too large");
  fir_rows_warp_kernel<<<ceil_div_u(warps * 32, kThreads), kThreads, 0, stream>>>(
      static_cast<const bf16 *>(input), filter, filter_is_f32, static_cast<const bf16 *>(bias), multiply_bias,
      cache, static_cast<bf16 *>(output), length, channels, channels / groups, static_cast<int>(taps),
      static_cast<int>(cache_length), cross_correlation);
  const int status = check_launch("FIR step kernel");
  if (status != kOk) return status;
  return update_history(input, cache, length, channels, taps - 1, false, stream);
}

}  // namespace evob
