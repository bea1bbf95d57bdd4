// Long-implicit (HCL) Hyena operator: y = x2 * (h * u + D u) with
// u = bf16(x1 * v) and the per-channel modal filter
// h[c,t] = sum_m R[c,m] exp(log_pole[c,m] t).
//
// Upstream materialises h and convolves with an n = 2T FFT, then recovers the
// decode state with one complex FFT per (channel, mode)
// (src/cuda/hyena.cu:562-660, 1262-1456, 1994-2124).  Because the filter is a
// sum of first-order modes, the same convolution is a linear recurrence
// s_m[t] = p_m s_m[t-1] + u[t], y[t] = sum_m R_m s_m[t]; here it runs as a
// three-kernel chunked scan that is linear in T, needs T*C*modes/segment
// floats of scratch instead of FFT planes, and yields the decode state for free:
//   1. per (segment, channel pair): end state of the segment from zero,
//   2. per (channel, mode): serial carry over segments (p^S scaling),
//   3. per (segment, channel pair): replay from the carried state, read out,
//      add the direct term, post-gate, store.
// The four BF16 roundings of the upstream epilogue are kept for initial
// prefill; continuation chunks keep upstream's single rounding
// (src/cuda/hyena.cu:534-560).  modal_decode keeps the pinned decode order
// (separate multiply/add, 32-lane zero-padded tree; src/cuda/hyena.cu:718-761).
#include <mutex>
#include <string>

#include "common.cuh"
#include "ops_internal.hpp"
#include "projection_featurizer.cuh"

namespace evob {
namespace {

constexpr int kThreads = 128;

struct ModalParams {
  const bf16 *x2, *x1, *value, *projection, *short_filter, *direct;
  const float *log_poles, *residues;
  bf16 *output, *pregate;
  float *state;    // [width, modes]
  float *scratch;  // [segments, width, modes]
  // optional [length, width] packed (u | x2 << 16) words: written by the
  // projection-fed local pass, read by the output pass instead of featurizing again
  std::uint32_t *words;
  int length, row_begin, width, segment, segments, pairs;
  bool continue_from_state;
};

// Streams one channel pair through time, yielding the featurized gate values.
template <bool kFromProjection>
struct PairReader {
  const ModalParams &p;
  int c0;
  float prev1[6], prev2[6];  // raw projection rows t-1, t-2 (x2a,x1a,va,x2b,x1b,vb)
  float sw[6][3];            // featurizer taps per stream of the pair

  __device__ __forceinline__ PairReader(const ModalParams &params, const int channel)
      : p(params), c0(channel) {}

  __device__ __forceinline__ void load_row(const int t, float (&row)[6]) const {
    if (t < 0) {
#pragma unroll
      for (int i = 0; i < 6; ++i) row[i] = 0.0F;
      return;
    }
    const std::uint32_t *const words = reinterpret_cast<const std::uint32_t *>(
        p.projection + static_cast<std::size_t>(t) * p.width * 3 + c0 * 3);
#pragma unroll
    for (int w = 0; w < 3; ++w) {
      const std::uint32_t word = words[w];
      row[2 * w] = __uint_as_float(word << 16U);
      row[2 * w + 1] = __uint_as_float(word & 0xffff0000U);
    }
  }

  __device__ __forceinline__ void start(const int t0) {
    if constexpr (kFromProjection) {
#pragma unroll
      for (int s = 0; s < 6; ++s)
#pragma unroll
        for (int j = 0; j < 3; ++j)
          sw[s][j] = bf2f(p.short_filter[(static_cast<std::size_t>(c0) * 3 + s) * 3 + j]);
      load_row(t0 - 1, prev1);
      load_row(t0 - 2, prev2);
    }
  }

  // Loads issued for kBatch consecutive rows before any of them is consumed:
  // the recurrence is a serial dependency chain, so memory latency has to be
  // covered by independent loads in flight, not by the chain.
  static constexpr int kBatch = 8;

  __device__ __forceinline__ void fetch(const int t, const int limit, const bool want_x2,
                                        std::uint32_t (&raw)[kBatch][3]) const {
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      const int row = t + i;
      raw[i][0] = raw[i][1] = raw[i][2] = 0U;
      if (row < limit) {
        if constexpr (kFromProjection) {
          const std::uint32_t *const words = reinterpret_cast<const std::uint32_t *>(
              p.projection + static_cast<std::size_t>(row) * p.width * 3 + c0 * 3);
          raw[i][0] = __ldg(words);
          raw[i][1] = __ldg(words + 1);
          raw[i][2] = __ldg(words + 2);
        } else {
          const std::size_t index = static_cast<std::size_t>(row) * p.width + c0;
          raw[i][0] = __ldg(reinterpret_cast<const std::uint32_t *>(p.x1 + index));
          raw[i][1] = __ldg(reinterpret_cast<const std::uint32_t *>(p.value + index));
          if (want_x2) raw[i][2] = __ldg(reinterpret_cast<const std::uint32_t *>(p.x2 + index));
        }
      }
    }
  }

  // Consumes one fetched row: u for both channels and the x2 gate.
  __device__ __forceinline__ void step(const std::uint32_t (&words)[3], float &u0, float &u1,
                                       float &g0, float &g1) {
    if constexpr (kFromProjection) {
      float row[6], z[6];
#pragma unroll
      for (int w = 0; w < 3; ++w) {
        row[2 * w] = __uint_as_float(words[w] << 16U);
        row[2 * w + 1] = __uint_as_float(words[w] & 0xffff0000U);
      }
#pragma unroll
      for (int s = 0; s < 6; ++s) {
        float a = 0.0F;
        a = fmaf(prev2[s], sw[s][0], a);
        a = fmaf(prev1[s], sw[s][1], a);
        a = fmaf(row[s], sw[s][2], a);
        z[s] = rbf(a);
        prev2[s] = prev1[s];
        prev1[s] = row[s];
      }
      u0 = rbf(z[1] * z[2]);
      u1 = rbf(z[4] * z[5]);
      g0 = z[0];
      g1 = z[3];
    } else {
      const std::uint32_t a = words[0], b = words[1], g = words[2];
      u0 = rbf(__uint_as_float(a << 16U) * __uint_as_float(b << 16U));
      u1 = rbf(__uint_as_float(a & 0xffff0000U) * __uint_as_float(b & 0xffff0000U));
      g0 = __uint_as_float(g << 16U);
      g1 = __uint_as_float(g & 0xffff0000U);
    }
  }
};

template <int kModes, bool kFromProjection>
__global__ void __launch_bounds__(kThreads)
modal_local_kernel(const ModalParams p) {
  const int index = blockIdx.x * kThreads + threadIdx.x;
  const int pair = index % p.pairs;
  const int seg = index / p.pairs;
  if (seg >= p.segments) return;
  const int c0 = pair * 2;
  if (c0 >= p.width) return;
  float pole[2][kModes], state[2][kModes];
#pragma unroll
  for (int c = 0; c < 2; ++c)
#pragma unroll
    for (int m = 0; m < kModes; ++m) {
      pole[c][m] = expf(p.log_poles[static_cast<std::size_t>(c0 + c) * kModes + m]);
      state[c][m] = 0.0F;
    }
  const int t0 = p.row_begin + seg * p.segment;
  const int t1 = min(t0 + p.segment, p.length);
  PairReader<kFromProjection> reader(p, c0);
  reader.start(t0);
  constexpr int kBatch = PairReader<kFromProjection>::kBatch;
  for (int t = t0; t < t1; t += kBatch) {
    std::uint32_t raw[kBatch][3];
    reader.fetch(t, t1, false, raw);
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      if (t + i < t1) {
        float u0, u1, g0, g1;
        reader.step(raw[i], u0, u1, g0, g1);
#pragma unroll
        for (int m = 0; m < kModes; ++m) {
          state[0][m] = fmaf(pole[0][m], state[0][m], u0);
          state[1][m] = fmaf(pole[1][m], state[1][m], u1);
        }
      }
    }
  }
  float *const out = p.scratch + (static_cast<std::size_t>(seg) * p.width + c0) * kModes;
#pragma unroll
  for (int c = 0; c < 2; ++c)
#pragma unroll
    for (int m = 0; m < kModes; ++m) out[c * kModes + m] = state[c][m];
}

// scratch[seg] holds the segment-local end state on entry and the state carried
// INTO the segment on exit; the state after the last segment goes to p.state.
__global__ void modal_carry_kernel(const ModalParams p, const int modes) {
  const int index = blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= p.width * modes) return;
  const float log_pole = p.log_poles[index];
  const float full_decay = expf(log_pole * static_cast<float>(p.segment));
  float carry = (p.continue_from_state && p.state != nullptr) ? p.state[index] : 0.0F;
  const std::size_t stride = static_cast<std::size_t>(p.width) * modes;
  // The chain over segments is serial; its loads are not, so they are issued
  // a batch at a time ahead of the dependent arithmetic.
  constexpr int kAhead = 16;
  for (int seg0 = 0; seg0 < p.segments; seg0 += kAhead) {
    float local[kAhead];
#pragma unroll
    for (int i = 0; i < kAhead; ++i)
      local[i] = seg0 + i < p.segments ? __ldcg(p.scratch + (seg0 + i) * stride + index) : 0.0F;
#pragma unroll
    for (int i = 0; i < kAhead; ++i) {
      const int seg = seg0 + i;
      if (seg < p.segments) {
        p.scratch[seg * stride + index] = carry;
        const int span = min(p.segment, p.length - p.row_begin - seg * p.segment);
        const float decay =
            span == p.segment ? full_decay : expf(log_pole * static_cast<float>(span));
        carry = fmaf(decay, carry, local[i]);
      }
    }
  }
  if (p.state != nullptr) p.state[index] = carry;
}

template <int kModes, bool kFromProjection>
__global__ void __launch_bounds__(kThreads)
modal_output_kernel(const ModalParams p) {
  const int index = blockIdx.x * kThreads + threadIdx.x;
  const int pair = index % p.pairs;
  const int seg = index / p.pairs;
  if (seg >= p.segments) return;
  const int c0 = pair * 2;
  if (c0 >= p.width) return;
  float pole[2][kModes], residue[2][kModes], state[2][kModes];
  const float *const carried =
      p.scratch + (static_cast<std::size_t>(seg) * p.width + c0) * kModes;
#pragma unroll
  for (int c = 0; c < 2; ++c)
#pragma unroll
    for (int m = 0; m < kModes; ++m) {
      const std::size_t q = static_cast<std::size_t>(c0 + c) * kModes + m;
      pole[c][m] = expf(p.log_poles[q]);
      residue[c][m] = p.residues[q];
      state[c][m] = carried[c * kModes + m];
    }
  const float direct0 = bf2f(p.direct[c0]);
  const float direct1 = bf2f(p.direct[c0 + 1]);
  const int t0 = p.row_begin + seg * p.segment;
  const int t1 = min(t0 + p.segment, p.length);
  PairReader<kFromProjection> reader(p, c0);
  reader.start(t0);
  constexpr int kBatch = PairReader<kFromProjection>::kBatch;
  for (int tb = t0; tb < t1; tb += kBatch) {
   std::uint32_t raw[kBatch][3];
   reader.fetch(tb, t1, true, raw);
#pragma unroll
   for (int i = 0; i < kBatch; ++i) {
    const int t = tb + i;
    if (t >= t1) break;
    float u[2], g[2];
    reader.step(raw[i], u[0], u[1], g[0], g[1]);
    float result[2];
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      float partial[4] = {0.0F, 0.0F, 0.0F, 0.0F};
#pragma unroll
      for (int m = 0; m < kModes; ++m) {
        state[c][m] = fmaf(pole[c][m], state[c][m], u[c]);
        partial[m % 4] = fmaf(residue[c][m], state[c][m], partial[m % 4]);
      }
      const float modal = ((partial[0] + partial[1]) + partial[2]) + partial[3];
      const float direct = c == 0 ? direct0 : direct1;
      if (p.continue_from_state) {
        result[c] = g[c] * fmaf(direct, u[c], modal);
      } else {
        const float mixed = rbf(rbf(modal) + rbf(direct * u[c]));
        result[c] = mixed * g[c];
      }
    }
    const std::size_t offset = static_cast<std::size_t>(t) * p.width + c0;
    *reinterpret_cast<std::uint32_t *>(p.output + offset) =
        pack_bf16x2(result[0], result[1]);
    if (p.pregate != nullptr)
      *reinterpret_cast<std::uint32_t *>(p.pregate + offset) =
          (__float_as_uint(u[0]) >> 16U) | (__float_as_uint(u[1]) & 0xffff0000U);
   }
  }
}

__global__ void modal_decode_kernel(const bf16 *__restrict__ x2,
                                    const bf16 *__restrict__ x1,
                                    const bf16 *__restrict__ value,
                                    const bf16 *__restrict__ direct,
                                    const float *__restrict__ log_poles,
                                    const float *__restrict__ residues,
                                    float *__restrict__ state,
                                    bf16 *__restrict__ pregate,
                                    bf16 *__restrict__ output, const int width,
                                    const int modes) {
  const int channel = blockIdx.x * blockDim.x + threadIdx.x;
  if (channel >= width) return;
  const bf16 gated_bf16 = f2bf(bf2f(x1[channel]) * bf2f(value[channel]));
  if (pregate != nullptr) pregate[channel] = gated_bf16;
  const float gated = bf2f(gated_bf16);
  float terms[32];
#pragma unroll
  for (int lane = 0; lane < 32; ++lane) terms[lane] = 0.0F;
#pragma unroll
  for (int mode = 0; mode < 32; ++mode) {
    if (mode < modes) {
      const std::size_t q = static_cast<std::size_t>(channel) * modes + mode;
      const float updated =
          __fadd_rn(__fmul_rn(expf(log_poles[q]), state[q]), gated);
      state[q] = updated;
      terms[mode] = __fmul_rn(residues[q], updated);
    }
  }
#pragma unroll
  for (int offset = 16; offset != 0; offset /= 2)
#pragma unroll
    for (int lane = 0; lane < 32; ++lane)
      if (lane < 32 - offset) terms[lane] = __fadd_rn(terms[lane], terms[lane + offset]);
  const float direct_product = rbf(bf2f(direct[channel]) * gated);
  const float mixed = __fadd_rn(terms[0], direct_product);
  output[channel] = f2bf(__fmul_rn(bf2f(x2[channel]), mixed));
}

// ---------------------------------------------------------------- tiled scan
// The same local / output passes with the inputs staged through shared memory.
// A CTA owns 64 channels x kLanes consecutive segments and walks them in slabs
// of kSlab rows: cp.async copies the next slab's rows (double buffered) while
// the current one is featurized cooperatively with 128-bit accesses - one
// (segment lane, row, 8-channel chunk) per thread - into packed (u, x2) words;
// then every thread advances the recurrence of ONE channel of one segment lane
// over the slab's rows, reading its word per row from shared memory, and the
// finished rows leave through a shared tile with 128-bit stores.  No thread
// waits on a global load of its own, and the per-thread state is 3*modes
// registers instead of 6*modes, which is what lets two CTAs share an SM.
constexpr int kScanThreads = 256;
constexpr int kTileChannels = 64;
constexpr int kLanes = 4;
constexpr int kSlab = 8;
constexpr int kProjRowBytes = kTileChannels * 3 * 2;                      // 384
constexpr int kProjStageBytes = kLanes * (kSlab + 2) * kProjRowBytes;     // 15360
constexpr int kPlainRowBytes = kTileChannels * 2;                         // 128
constexpr int kPlainStageBytes = 3 * kLanes * kSlab * kPlainRowBytes;     // 12288
constexpr int kWordTileBytes = kLanes * kSlab * kTileChannels * 4;        // 8192
constexpr int kOutTileBytes = kLanes * kSlab * kTileChannels * 2;         // 4096
constexpr int kWeightBytes = 8 * 36 * 4;                                  // 1152

template <bool kFromProjection>
constexpr int tiled_smem_bytes() {
  return 2 * (kFromProjection ? kProjStageBytes : kPlainStageBytes) + kWordTileBytes + kOutTileBytes +
         (kFromProjection ? kWeightBytes : 0);
}

__device__ __forceinline__ void async_copy16(void *shared, const void *global, const bool valid) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(
                   static_cast<std::uint32_t>(__cvta_generic_to_shared(shared))),
               "l"(global), "r"(valid ? 16U : 0U)
               : "memory");
}

// A thread's share of the 16-byte copies of a slab; the (lane, row, chunk) a
// thread copies is the same for every slab, so only the row bound is checked
// per slab.
template <bool kFromProjection, bool kNeedGate>
struct ModalCopies {
  static constexpr int kTotal =
      kFromProjection ? kLanes * (kSlab + 2) * 24 : (kNeedGate ? 3 : 2) * kLanes * kSlab * 8;
  static constexpr int kPerThread = (kTotal + kScanThreads - 1) / kScanThreads;
  const bf16 *source[kPerThread];   // address of the copy for slab 0 (may be out of range: see row)
  std::uint32_t destination[kPerThread];
  int row[kPerThread];              // time of the copy for slab 0; a huge value when unused

  __device__ __forceinline__ void plan(const ModalParams &p, const int seg0, const int c_tile) {
#pragma unroll
    for (int k = 0; k < kPerThread; ++k) {
      const int item = threadIdx.x + k * kScanThreads;
      int lane, j, t, column_elements;
      const bf16 *base;
      std::size_t pitch;
      bool used = item < kTotal;
      if constexpr (kFromProjection) {
        const int chunk = item % 24;
        j = (item / 24) % (kSlab + 2);
        lane = item / (24 * (kSlab + 2));
        t = p.row_begin + (seg0 + lane) * p.segment + j - 2;
        pitch = static_cast<std::size_t>(p.width) * 3;
        column_elements = c_tile * 3 + chunk * 8;
        used = used && static_cast<std::size_t>(column_elements) + 8 <= pitch;
        base = p.projection;
        destination[k] = static_cast<std::uint32_t>((lane * (kSlab + 2) + j) * kProjRowBytes + chunk * 16);
      } else {
        const int chunk = item % 8;
        j = (item / 8) % kSlab;
        lane = (item / (8 * kSlab)) % kLanes;
        const int stream = item / (8 * kSlab * kLanes);
        t = p.row_begin + (seg0 + lane) * p.segment + j;
        pitch = static_cast<std::size_t>(p.width);
        column_elements = c_tile + chunk * 8;
        used = used && column_elements < p.width;
        base = stream == 0 ? p.x1 : (stream == 1 ? p.value : p.x2);
        destination[k] =
            static_cast<std::uint32_t>(((stream * kLanes + lane) * kSlab + j) * kPlainRowBytes + chunk * 16);
      }
      used = used && seg0 + lane < p.segments;
      row[k] = used ? t : 0x40000000;
      source[k] = base + static_cast<long long>(t) * static_cast<long long>(pitch) + column_elements;
    }
  }
  __device__ __forceinline__ void issue(const ModalParams &p, unsigned char *stage, const int slab) const {
    const std::uint32_t base = static_cast<std::uint32_t>(__cvta_generic_to_shared(stage));
    const std::size_t advance = static_cast<std::size_t>(slab) * kSlab *
                                (kFromProjection ? static_cast<std::size_t>(p.width) * 3 : p.width);
#pragma unroll
    for (int k = 0; k < kPerThread; ++k) {
      if (threadIdx.x + k * kScanThreads >= kTotal) break;
      const bool valid = static_cast<unsigned int>(row[k] + slab * kSlab) < static_cast<unsigned int>(p.length);
      const bf16 *const from = valid ? source[k] + advance : p.direct;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(base + destination[k]), "l"(from),
                   "r"(valid ? 16U : 0U)
                   : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
};

template <int kModes, bool kFromProjection, bool kOutput>
__global__ void __launch_bounds__(kScanThreads, 2)
modal_tiled_kernel(const ModalParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int kStageBytes = kFromProjection ? kProjStageBytes : kPlainStageBytes;
  unsigned char *const stages = smem;
  std::uint32_t *const words = reinterpret_cast<std::uint32_t *>(smem + 2 * kStageBytes);
  unsigned short *const out_tile = reinterpret_cast<unsigned short *>(smem + 2 * kStageBytes + kWordTileBytes);
  std::uint32_t *const weights =
      reinterpret_cast<std::uint32_t *>(smem + 2 * kStageBytes + kWordTileBytes + kOutTileBytes);
  const int seg0 = blockIdx.x * kLanes;
  const int c_tile = blockIdx.y * kTileChannels;
  const int lane = threadIdx.x / kTileChannels;  // segment lane of both roles
  const int column = threadIdx.x % kTileChannels;

  // ---- scan role: channel `channel` of segment seg0 + lane
  const int channel = c_tile + column;
  const int seg = seg0 + lane;
  const bool scans = channel < p.width && seg < p.segments;
  const int t0 = p.row_begin + seg * p.segment;
  const int t1 = min(t0 + p.segment, p.length);
  float pole[kModes], residue[kModes], state[kModes];
  float direct = 0.0F;
#pragma unroll
  for (int m = 0; m < kModes; ++m) {
    pole[m] = residue[m] = state[m] = 0.0F;
    if (scans) {
      const std::size_t q = static_cast<std::size_t>(channel) * kModes + m;
      pole[m] = expf(p.log_poles[q]);
      if constexpr (kOutput) {
        residue[m] = p.residues[q];
        state[m] = p.scratch[(static_cast<std::size_t>(seg) * p.width + channel) * kModes + m];
      }
    }
  }
  if constexpr (kOutput)
    if (scans) direct = bf2f(p.direct[channel]);

  // ---- featurize / store role: row item_row, channels item_c0 .. +8 of the lane
  const int item_chunk = threadIdx.x % 8;
  const int item_row = (threadIdx.x / 8) % kSlab;
  const int item_c0 = c_tile + item_chunk * 8;
  const bool item_ok = item_c0 < p.width && seg < p.segments;
  if constexpr (kFromProjection) {
    if (threadIdx.x < 72) {
      const int chunk = threadIdx.x / 9, part = threadIdx.x % 9;
      uint4 v = make_uint4(0U, 0U, 0U, 0U);
      if (c_tile + chunk * 8 < p.width)
        v = __ldg(reinterpret_cast<const uint4 *>(p.short_filter +
                                                  static_cast<std::size_t>(c_tile + chunk * 8) * 9) + part);
      *reinterpret_cast<uint4 *>(weights + chunk * 36 + part * 4) = v;
    }
  }
  ModalCopies<kFromProjection, kOutput> copies;
  copies.plan(p, seg0, c_tile);
  const int slabs = p.segment / kSlab;
  copies.issue(p, stages, 0);
  for (int slab = 0; slab < slabs; ++slab) {
    const unsigned char *const stage = stages + (slab & 1) * kStageBytes;
    if (slab + 1 < slabs) {
      copies.issue(p, stages + ((slab + 1) & 1) * kStageBytes, slab + 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    {  // featurize one (lane, row, chunk) item into packed words: u low, x2 high
      std::uint32_t u[4], g[4] = {0U, 0U, 0U, 0U};
      if constexpr (kFromProjection) {
        const unsigned char *const base =
            stage + (lane * (kSlab + 2) + item_row) * kProjRowBytes + item_chunk * 48;
        const unsigned char *const history[3] = {base, base + kProjRowBytes, base + 2 * kProjRowBytes};
        PackedTaps taps;
        taps.load_shared(weights + item_chunk * 36);
        if constexpr (kOutput) {
          featurize_chunk<true>(history, taps, u, g);
        } else {
          // the local pass needs only u, unless it also leaves the words for the output pass
          if (p.words != nullptr) featurize_chunk<true>(history, taps, u, g);
          else featurize_chunk<false>(history, taps, u, g);
        }
      } else {
        const unsigned char *const base = stage + (lane * kSlab + item_row) * kPlainRowBytes + item_chunk * 16;
        Bf16x8 a, b;
        a.raw = *reinterpret_cast<const uint4 *>(base);
        b.raw = *reinterpret_cast<const uint4 *>(base + kLanes * kSlab * kPlainRowBytes);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          u[j] = round_pair_bf16(a.get(2 * j) * b.get(2 * j), a.get(2 * j + 1) * b.get(2 * j + 1));
        if constexpr (kOutput) {
          const uint4 c = *reinterpret_cast<const uint4 *>(base + 2 * kLanes * kSlab * kPlainRowBytes);
          g[0] = c.x; g[1] = c.y; g[2] = c.z; g[3] = c.w;
        }
      }
      uint4 *const destination = reinterpret_cast<uint4 *>(
          words + (lane * kSlab + item_row) * kTileChannels + item_chunk * 8);
      // word of channel c = u_c | x2_c << 16
      destination[0] = make_uint4(__byte_perm(u[0], g[0], 0x5410), __byte_perm(u[0], g[0], 0x7632),
                                  __byte_perm(u[1], g[1], 0x5410), __byte_perm(u[1], g[1], 0x7632));
      destination[1] = make_uint4(__byte_perm(u[2], g[2], 0x5410), __byte_perm(u[2], g[2], 0x7632),
                                  __byte_perm(u[3], g[3], 0x5410), __byte_perm(u[3], g[3], 0x7632));
      if constexpr (kFromProjection && !kOutput) {
        const int t = t0 + slab * kSlab + item_row;
        if (p.words != nullptr && item_ok && t < t1) {
          uint4 *const out = reinterpret_cast<uint4 *>(p.words + static_cast<std::size_t>(t) * p.width + item_c0);
          out[0] = destination[0];
          out[1] = destination[1];
        }
      }
      if constexpr (kOutput) {
        const int t = t0 + slab * kSlab + item_row;
        if (p.pregate != nullptr && item_ok && t < t1)
          *reinterpret_cast<uint4 *>(p.pregate + static_cast<std::size_t>(t) * p.width + item_c0) =
              make_uint4(u[0], u[1], u[2], u[3]);
      }
    }
    __syncthreads();
    if (scans) {
      const int first = t0 + slab * kSlab;
      const std::uint32_t *const my_words = words + lane * kSlab * kTileChannels + column;
      unsigned short *const my_out = out_tile + lane * kSlab * kTileChannels + column;
      // rows of this slab inside the segment (all of them except in the last segment)
      const int live = min(kSlab, t1 - first);
#pragma unroll
      for (int r = 0; r < kSlab; ++r) {
        if (r < live) {
          const std::uint32_t word = my_words[r * kTileChannels];
          const float u = __uint_as_float(word << 16U);
          if constexpr (kOutput) {
            const float g = __uint_as_float(word & 0xffff0000U);
            float partial[4] = {0.0F, 0.0F, 0.0F, 0.0F};
#pragma unroll
            for (int m = 0; m < kModes; ++m) {
              state[m] = fmaf(pole[m], state[m], u);
              partial[m % 4] = fmaf(residue[m], state[m], partial[m % 4]);
            }
            const float modal = ((partial[0] + partial[1]) + partial[2]) + partial[3];
            float result;
            if (p.continue_from_state)
              result = g * fmaf(direct, u, modal);
            else
              result = rbf(rbf(modal) + rbf(direct * u)) * g;
            my_out[r * kTileChannels] = static_cast<unsigned short>(__float_as_uint(rbf(result)) >> 16U);
          } else {
#pragma unroll
            for (int m = 0; m < kModes; ++m) state[m] = fmaf(pole[m], state[m], u);
          }
        }
      }
    }
    if constexpr (kOutput) {
      __syncthreads();
      const int t = t0 + slab * kSlab + item_row;
      if (item_ok && t < t1)
        *reinterpret_cast<uint4 *>(p.output + static_cast<std::size_t>(t) * p.width + item_c0) =
            *reinterpret_cast<const uint4 *>(out_tile + (lane * kSlab + item_row) * kTileChannels + item_chunk * 8);
    }
  }
  if constexpr (!kOutput) {
    if (scans) {
      float *const out = p.scratch + (static_cast<std::size_t>(seg) * p.width + channel) * kModes;
#pragma unroll
      for (int m = 0; m < kModes; ++m) out[m] = state[m];
    }
  }
}

// Output pass from the stored (u, x2) words: no featurizer, no raw staging -
// the words of the next slab are copied in while this one is scanned.

template <int kModes>
__global__ void __launch_bounds__(kScanThreads, 3)
modal_words_output_kernel(const ModalParams p) {
  __shared__ __align__(16) std::uint32_t stages[2][kLanes * kSlab * kTileChannels];
  __shared__ __align__(16) unsigned short out_tile[kLanes * kSlab * kTileChannels];
  const int seg0 = blockIdx.x * kLanes;
  const int c_tile = blockIdx.y * kTileChannels;
  const int lane = threadIdx.x / kTileChannels;
  const int column = threadIdx.x % kTileChannels;
  const int channel = c_tile + column;
  const int seg = seg0 + lane;
  const bool scans = channel < p.width && seg < p.segments;
  const int t0 = p.row_begin + seg * p.segment;
  const int t1 = min(t0 + p.segment, p.length);
  float pole[kModes], residue[kModes], state[kModes];
  float direct = 0.0F;
#pragma unroll
  for (int m = 0; m < kModes; ++m) {
    pole[m] = residue[m] = state[m] = 0.0F;
    if (scans) {
      const std::size_t q = static_cast<std::size_t>(channel) * kModes + m;
      pole[m] = expf(p.log_poles[q]);
      residue[m] = p.residues[q];
      state[m] = p.scratch[(static_cast<std::size_t>(seg) * p.width + channel) * kModes + m];
    }
  }
  if (scans) direct = bf2f(p.direct[channel]);
  // copy / store role: row item_row of the lane, two 16-byte chunks (8 channels) per thread
  const int item_chunk = threadIdx.x % 8;
  const int item_row = (threadIdx.x / 8) % kSlab;
  const int item_c0 = c_tile + item_chunk * 8;
  const bool item_ok = item_c0 < p.width && seg < p.segments;
  const auto issue = [&](const int slab, std::uint32_t *const stage) {
    const int t = t0 + slab * kSlab + item_row;
    const bool valid = item_ok && t < t1;
    const std::uint32_t *const source =
        valid ? p.words + static_cast<std::size_t>(t) * p.width + item_c0 : p.words;
    std::uint32_t *const target = stage + (lane * kSlab + item_row) * kTileChannels + item_chunk * 8;
    async_copy16(target, source, valid);
    async_copy16(target + 4, source + 4, valid);
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  const int slabs = p.segment / kSlab;
  issue(0, stages[0]);
  for (int slab = 0; slab < slabs; ++slab) {
    const std::uint32_t *const stage = stages[slab & 1];
    if (slab + 1 < slabs) {
      issue(slab + 1, stages[(slab + 1) & 1]);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    if (p.pregate != nullptr) {
      const int t = t0 + slab * kSlab + item_row;
      if (item_ok && t < t1) {
        const std::uint32_t *const w = stage + (lane * kSlab + item_row) * kTileChannels + item_chunk * 8;
        *reinterpret_cast<uint4 *>(p.pregate + static_cast<std::size_t>(t) * p.width + item_c0) =
            make_uint4(__byte_perm(w[0], w[1], 0x5410), __byte_perm(w[2], w[3], 0x5410),
                       __byte_perm(w[4], w[5], 0x5410), __byte_perm(w[6], w[7], 0x5410));
      }
    }
    if (scans) {
      const std::uint32_t *const my_words = stage + lane * kSlab * kTileChannels + column;
      unsigned short *const my_out = out_tile + lane * kSlab * kTileChannels + column;
      const int live = min(kSlab, t1 - (t0 + slab * kSlab));
#pragma unroll
      for (int r = 0; r < kSlab; ++r) {
        if (r < live) {
          const std::uint32_t word = my_words[r * kTileChannels];
          const float u = __uint_as_float(word << 16U);
          const float g = __uint_as_float(word & 0xffff0000U);
          float partial[4] = {0.0F, 0.0F, 0.0F, 0.0F};
#pragma unroll
          for (int m = 0; m < kModes; ++m) {
            state[m] = fmaf(pole[m], state[m], u);
            partial[m % 4] = fmaf(residue[m], state[m], partial[m % 4]);
          }
          const float modal = ((partial[0] + partial[1]) + partial[2]) + partial[3];
          float result;
          if (p.continue_from_state)
            result = g * fmaf(direct, u, modal);
          else
            result = rbf(rbf(modal) + rbf(direct * u)) * g;
          my_out[r * kTileChannels] = static_cast<unsigned short>(__float_as_uint(rbf(result)) >> 16U);
        }
      }
    }
    __syncthreads();
    {
      const int t = t0 + slab * kSlab + item_row;
      if (item_ok && t < t1)
        *reinterpret_cast<uint4 *>(p.output + static_cast<std::size_t>(t) * p.width + item_c0) =
            *reinterpret_cast<const uint4 *>(out_tile + (lane * kSlab + item_row) * kTileChannels + item_chunk * 8);
    }
    // the next round's scan writes out_tile only after its own barrier; the stage buffer
    // refilled next round is the one scanned two rounds ago
  }
}

bool tiled_scan_applies(const ModalParams &p, const bool from_projection) {
  const auto aligned = [](const void *q) { return (reinterpret_cast<std::uintptr_t>(q) & 15U) == 0; };
  if (p.width % 8 != 0 || p.segment % kSlab != 0 || !aligned(p.output) ||
      (p.pregate != nullptr && !aligned(p.pregate)))
    return false;
  return from_projection ? aligned(p.projection) && aligned(p.short_filter)
                         : aligned(p.x1) && aligned(p.value) && aligned(p.x2);
}

template <int kModes, bool kFromProjection>
int launch_tiled(const ModalParams &p, cudaStream_t stream) {
  constexpr int smem = tiled_smem_bytes<kFromProjection>();
  static_assert(smem <= 48 * 1024, "the tiled modal scan is sized for the default shared-memory limit");
  const dim3 grid(ceil_div_u(p.segments, kLanes), ceil_div_u(p.width, kTileChannels));
  if (grid.y > 65535) return fail(kInvalidArgument, "modal prefill is too wide");
  modal_tiled_kernel<kModes, kFromProjection, false><<<grid, kScanThreads, smem, stream>>>(p);
  int status = check_launch("modal segment kernel");
  if (status != kOk) return status;
  modal_carry_kernel<<<ceil_div_u(static_cast<std::size_t>(p.width) * kModes, 256), 256, 0, stream>>>(p, kModes);
  status = check_launch("modal carry kernel");
  if (status != kOk) return status;
  if (kFromProjection && p.words != nullptr)
    modal_words_output_kernel<kModes><<<grid, kScanThreads, 0, stream>>>(p);
  else
    modal_tiled_kernel<kModes, kFromProjection, true><<<grid, kScanThreads, smem, stream>>>(p);
  return check_launch("modal output kernel");
}

int pick_segment(const std::size_t length, const std::size_t width) {
  // Largest segment that still yields >= ~200k threads; shorter segments cost
  // more carry scratch, longer ones starve the SMs.
  const std::size_t pairs = width / 2;
  for (const int segment : {256, 128, 64, 32, 16}) {
    const std::size_t segments = (length + segment - 1) / segment;
    if (segments * pairs >= 200000) return segment;
  }
  return 16;
}

template <int kModes>
int launch_modal(const ModalParams &p, const bool from_projection,
                 cudaStream_t stream) {
  if (tiled_scan_applies(p, from_projection))
    return from_projection ? launch_tiled<kModes, true>(p, stream) : launch_tiled<kModes, false>(p, stream);
  const std::size_t threads = static_cast<std::size_t>(p.segments) * p.pairs;
  const unsigned int grid = ceil_div_u(threads, kThreads);
  if (from_projection)
    modal_local_kernel<kModes, true><<<grid, kThreads, 0, stream>>>(p);
  else
    modal_local_kernel<kModes, false><<<grid, kThreads, 0, stream>>>(p);
  int status = check_launch("modal segment kernel");
  if (status != kOk) return status;
  modal_carry_kernel<<<ceil_div_u(static_cast<std::size_t>(p.width) * kModes, 256),
                       256, 0, stream>>>(p, kModes);
  status = check_launch("modal carry kernel");
  if (status != kOk) return status;
  if (from_projection)
    modal_output_kernel<kModes, true><<<grid, kThreads, 0, stream>>>(p);
  else
    modal_output_kernel<kModes, false><<<grid, kThreads, 0, stream>>>(p);
  return check_launch("modal output kernel");
}

}  // namespace

std::size_t modal_scratch_floats(const std::size_t length,
                                 const std::size_t width,
                                 const std::size_t modes) {
  if (length == 0) return 0;
  const std::size_t segment = pick_segment(length, width);
  // segment states, then one packed (u, x2) word per element for the projection-fed form
  return ((length + segment - 1) / segment) * width * modes + length * width;
}

int modal_prefill(const ModalArgs &a, cudaStream_t stream) {
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
  p.segment = pick_segment(a.length - a.row_begin, a.width);
  p.segments = static_cast<int>((a.length - a.row_begin + p.segment - 1) / p.segment);
  p.pairs = static_cast<int>(a.width / 2);
  p.continue_from_state = a.continue_from_state;
  // the words follow the segment states in the caller's scratch (sized by modal_scratch_floats
  // for the whole length; the segment states of this call take at most that function's first term)
  if (from_projection && a.width % 4 == 0) {
    const std::size_t full_segment = static_cast<std::size_t>(pick_segment(a.length, a.width));
    const std::size_t state_floats = ((a.length + full_segment - 1) / full_segment) * a.width * a.modes;
    if (static_cast<std::size_t>(p.segments) * a.width * a.modes <= state_floats)
      p.words = reinterpret_cast<std::uint32_t *>(a.scratch + state_floats);
  }
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
  if (status != kOk) return status;
  if (a.short_cache != nullptr && from_projection && a.short_taps > 1)
    status = fill_fir_cache(a.projection, a.short_cache, a.length, a.width * 3,
                            a.short_taps - 1, stream);
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
  if (a.projection != nullptr || a.x2 == nullptr || a.x1 == nullptr || a.value == nullptr ||
      a.direct == nullptr || a.log_poles == nullptr || a.residues == nullptr ||
      a.output == nullptr || a.width == 0 || a.width % 2 != 0 || a.modes == 0)
    return fail(kInvalidArgument, "allocation-free modal prefill arguments are invalid");
  if (a.continue_from_state && a.state == nullptr)
    return fail(kInvalidArgument, "modal continuation needs a state");
  if (a.length > 0x7fffff00U || a.width > 0x3fffffffU)
    return fail(kInvalidArgument, "modal prefill dimensions are too large");
  if (a.length == 0) return kOk;
  // Start from the segment length the allocating path would use and lengthen it
  // until the segment states fit the fixed array.
  std::size_t segment = static_cast<std::size_t>(pick_segment(a.length, a.width));
  const std::size_t per_segment = a.width * a.modes;
  while (((a.length + segment - 1) / segment) * per_segment > kStaticScratchFloats &&
         segment < a.length)
    segment *= 2;
  const std::size_t segments = (a.length + segment - 1) / segment;
  if (segments * per_segment > kStaticScratchFloats)
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
  p.segment = static_cast<int>(segment);
  p.segments = static_cast<int>(segments);
  p.pairs = static_cast<int>(a.width / 2);
  p.continue_from_state = a.continue_from_state;
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
  modal_decode_kernel<<<ceil_div_u(width, 128), 128, 0, stream>>>(
      static_cast<const bf16 *>(x2), static_cast<const bf16 *>(x1),
      static_cast<const bf16 *>(value), static_cast<const bf16 *>(direct),
      log_poles, residues, state, static_cast<bf16 *>(pregate),
      static_cast<bf16 *>(output), static_cast<int>(width),
      static_cast<int>(modes));
  return check_launch("modal decode kernel");
}

}  // namespace evob
