// Fused gated FIR prefill for the HCS (k=7) and HCM (k=128) Hyena mixers,
// fast path.  Same operator contract and rounding points as
// gated_fir_prefill_generic (hyena_fir.cu); this file is about moving the
// bytes well:
//
//  phase A  A 64-channel x (TT + halo) time tile of u = bf16(x1*v) and a
//           64 x TT tile of the x2 gate are built in shared memory with 128-bit
//           global loads.  When fed by the raw interleaved projection, its
//           columns of the tile are staged through shared memory in 32-row slabs
//           with cp.async (double buffered) and the 3-tap featurizer runs from
//           there, one (row, 8-channel chunk) per thread.
//  phase B  HCS and every odd configuration: CUDA-core FMAs, oldest tap first,
//           bit-identical to the generic kernel and to upstream's direct FIR.
//           HCM with BF16 filters shared by groups of 16k channels: the
//           convolution is a banded Toeplitz GEMM per group on warp-level BF16
//           MMAs (m16n8k16, F32 accumulation; products of BF16 operands are
//           exact, so only the summation order differs from the FMA chain):
//           Y[16 outputs x 16 channels] = H[16 x 144] . U[144 x 16], where
//           H[m][k] = h[128 + m - k] is the same nine fragments for every tile.
//  phase C  direct term, BF16 round, x2 post-gate, BF16 round, staged through
//           shared memory and stored with 128-bit writes.
//
// Filters of up to 8 taps whose groups are multiples of 4 channels (HCS) do not
// use tiles at all: gated_fir_stream_kernel keeps the whole sliding window in
// registers and reads every input once.
#include <algorithm>
#include <cstdlib>
#include <type_traits>

#include "common.cuh"
#include "ops_internal.hpp"
#include "projection_featurizer.cuh"

namespace evob {
namespace {

constexpr int kThreads = 256;
constexpr int kChannels = 64;           // channels per CTA
constexpr int kChunks = kChannels / 8;  // 16-byte chunks per tile row
constexpr int kRowBytes = kChannels * 2;
constexpr int kRun = 16;

struct Params {
  const bf16 *x2, *x1, *value, *projection, *short_filter, *direct;
  const void *filter;
  bf16 *output, *pregate;
  float *inner_cache;
  float *short_cache;  // streaming kernel only: F32 [3 width, 2] raw projection history
  int length, row_begin, width, taps, padded_taps, channels_per_group;
  bool filter_is_f32, cross_correlation;
};

// Tile rows are 128 bytes; 16-byte chunks are XOR-swizzled with the row so that
// ldmatrix and column-strided accesses are bank-conflict free.
__device__ __forceinline__ int tile_offset(const int row, const int chunk) {
  return row * kRowBytes + ((chunk ^ (row & 7)) << 4);
}
// Packed BF16 pair (channels 2p, 2p+1 of the tile) of one row.
__device__ __forceinline__ std::uint32_t tile_pair(const unsigned char *tile, const int row,
                                                   const int pair) {
  return *reinterpret_cast<const std::uint32_t *>(tile + tile_offset(row, pair >> 2) +
                                                  ((pair & 3) << 2));
}
__device__ __forceinline__ float lo(const std::uint32_t w) { return __uint_as_float(w << 16U); }
__device__ __forceinline__ float hi(const std::uint32_t w) {
  return __uint_as_float(w & 0xffff0000U);
}
__device__ __forceinline__ std::uint32_t pack_exact(const float a, const float b) {
  // both values are already BF16-representable
  return (__float_as_uint(a) >> 16U) | (__float_as_uint(b) & 0xffff0000U);
}
// i-th BF16 of a register array of packed pairs
template <int N>
__device__ __forceinline__ float element(const std::uint32_t (&words)[N], const int i) {
  return (i & 1) ? hi(words[i >> 1]) : lo(words[i >> 1]);
}

constexpr int kSlabRows = kThreads / kChunks;       // 32 featurized rows per slab
constexpr int kRawRowBytes = kChannels * 3 * 2;     // 384: the tile's columns of one projection row
constexpr int kRawSlabBytes = (kSlabRows + 2) * kRawRowBytes;
constexpr int kRawBytes = 2 * kRawSlabBytes;        // double buffer
constexpr int kSlabCopies = (kSlabRows + 2) * 24;   // 16-byte copies per slab
constexpr int kCopiesPerThread = (kSlabCopies + kThreads - 1) / kThreads;

// A thread's share of the 16-byte copies of a slab.  Which (row, chunk) a
// thread copies does not change from slab to slab, so everything but the time
// bound is worked out once.
struct SlabCopies {
  std::size_t source[kCopiesPerThread];    // element offset from row t_first of the slab
  std::uint32_t destination[kCopiesPerThread];  // byte offset inside a slab buffer
  int row[kCopiesPerThread];               // slab row, or a large negative number when unused

  __device__ __forceinline__ void plan(const Params &p, const int c_tile) {
    const std::size_t width3 = static_cast<std::size_t>(p.width) * 3;
#pragma unroll
    for (int k = 0; k < kCopiesPerThread; ++k) {
      const int item = threadIdx.x + k * kThreads;
      const int j = item / 24, chunk = item % 24;
      const std::size_t column = static_cast<std::size_t>(c_tile) * 3 + chunk * 8;
      const bool used = item < kSlabCopies && column + 8 <= width3;
      row[k] = used ? j : -0x40000000;
      source[k] = static_cast<std::size_t>(j) * width3 + column;
      destination[k] = static_cast<std::uint32_t>(j * kRawRowBytes + chunk * 16);
    }
  }
  // Rows outside [0, length) and unused copies arrive as zeros.  One commit group.
  __device__ __forceinline__ void issue(const Params &p, unsigned char *slab, const int t_first) const {
    const std::uint32_t base = static_cast<std::uint32_t>(__cvta_generic_to_shared(slab));
    const bf16 *const first = p.projection + static_cast<long long>(t_first) * (static_cast<long long>(p.width) * 3);
#pragma unroll
    for (int k = 0; k < kCopiesPerThread; ++k) {
      if (threadIdx.x + k * kThreads >= kSlabCopies) break;
      const bool valid = static_cast<unsigned int>(t_first + row[k]) < static_cast<unsigned int>(p.length);
      const bf16 *const from = valid ? first + source[k] : p.projection;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(base + destination[k]), "l"(from),
                   "r"(valid ? 16U : 0U)
                   : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
};

// Builds u rows [0, rows) (tile row r <-> time t_first + r) and, for tile rows
// >= gate_first_row, the x2 gate rows.  Also emits the optional pregate copy
// and the F32 decode history for rows this CTA owns (t >= t_own).
template <bool kProj>
__device__ __forceinline__ void build_tiles(const Params &p, unsigned char *u_tile,
                                            unsigned char *x2_tile, unsigned char *raw, const int rows,
                                            const int t_first, const int gate_first_row,
                                            const int t_own, const int c_tile, const bool first_of_window) {
  const int chunk = threadIdx.x % kChunks;
  const int c0 = c_tile + chunk * 8;
  const bool channel_ok = c0 < p.width;  // width is a multiple of 8
  const int real_halo = p.taps - 1;

  // u, g: packed BF16 pairs of channels (2j, 2j+1) of the chunk
  auto emit = [&](const int r, const int t, const std::uint32_t (&u)[4], const std::uint32_t (&g)[4],
                  const bool have_gate) {
    const uint4 packed = make_uint4(u[0], u[1], u[2], u[3]);
    *reinterpret_cast<uint4 *>(u_tile + tile_offset(r, chunk)) = packed;
    // The first CTA of a row window also owns the history rows it recomputes,
    // so that the decode history is complete even for windows shorter than it.
    const bool owns = t >= t_own || (first_of_window && t >= 0);
    if (owns && t < p.length && channel_ok) {
      if (p.pregate != nullptr && t >= t_own)
        *reinterpret_cast<uint4 *>(p.pregate + static_cast<std::size_t>(t) * p.width + c0) = packed;
      if (p.inner_cache != nullptr && real_halo > 0) {
        const int slot = t - (p.length - real_halo);
        if (slot >= 0) {
#pragma unroll
          for (int i = 0; i < 8; ++i)
            p.inner_cache[static_cast<std::size_t>(c0 + i) * real_halo + slot] = element(u, i);
        }
      }
    }
    if (have_gate)
      *reinterpret_cast<uint4 *>(x2_tile + tile_offset(r - gate_first_row, chunk)) =
          make_uint4(g[0], g[1], g[2], g[3]);
  };

  if constexpr (!kProj) {
    for (int r = threadIdx.x / kChunks; r < rows; r += kThreads / kChunks) {
      const int t = t_first + r;
      std::uint32_t u[4] = {}, g[4] = {};
      const bool live = channel_ok && t >= 0 && t < p.length;
      const bool have_gate = r >= gate_first_row;
      if (live) {
        const std::size_t index = static_cast<std::size_t>(t) * p.width + c0;
        Bf16x8 a, b;
        a.raw = __ldg(reinterpret_cast<const uint4 *>(p.x1 + index));
        b.raw = __ldg(reinterpret_cast<const uint4 *>(p.value + index));
#pragma unroll
        for (int j = 0; j < 4; ++j)
          u[j] = round_pair_bf16(a.get(2 * j) * b.get(2 * j), a.get(2 * j + 1) * b.get(2 * j + 1));
        if (have_gate) {
          const uint4 c = __ldg(reinterpret_cast<const uint4 *>(p.x2 + index));
          g[0] = c.x; g[1] = c.y; g[2] = c.z; g[3] = c.w;
        }
      }
      emit(r, t, u, g, have_gate);
    }
  } else {
    // The raw projection columns of the tile (64 channels x 3 streams = 384
    // contiguous bytes per row) are staged through shared memory in slabs of
    // kSlabRows rows with cp.async, double buffered, so the global loads of the
    // next slab are in flight while this one is featurized and no thread ever
    // waits on its own loads.  One (row, 8-channel chunk) item per thread.
    const int item_row = threadIdx.x / kChunks;
    PackedTaps taps;
    if (channel_ok) taps.load_global(p.short_filter, c0);
    SlabCopies copies;
    copies.plan(p, c_tile);
    const int slabs = (rows + kSlabRows - 1) / kSlabRows;
    copies.issue(p, raw, t_first - 2);
    for (int slab = 0; slab < slabs; ++slab) {
      const unsigned char *const buffer = raw + (slab & 1) * kRawSlabBytes;
      if (slab + 1 < slabs) {
        copies.issue(p, raw + ((slab + 1) & 1) * kRawSlabBytes, t_first + (slab + 1) * kSlabRows - 2);
        asm volatile("cp.async.wait_group 1;" ::: "memory");
      } else {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
      }
      __syncthreads();
      const int r = slab * kSlabRows + item_row;
      if (r < rows) {
        const int t = t_first + r;
        const bool live = channel_ok && t >= 0 && t < p.length;
        const bool have_gate = r >= gate_first_row;
        std::uint32_t u[4] = {}, g[4] = {};
        if (live) {
          const unsigned char *const base = buffer + item_row * kRawRowBytes + chunk * 48;
          const unsigned char *const history[3] = {base, base + kRawRowBytes, base + 2 * kRawRowBytes};
          featurize_chunk<true>(history, taps, u, g);
        }
        emit(r, t, u, g, have_gate);
      }
      __syncthreads();  // the other buffer is refilled at the top of the next round
    }
  }
}

__device__ __forceinline__ float filter_value(const void *filter, const bool is_f32,
                                              const std::size_t index) {
  return is_f32 ? static_cast<const float *>(filter)[index]
                : bf2f(static_cast<const bf16 *>(filter)[index]);
}

// Coalesced store of the finished TT x 64 tile (held in the x2 tile).
__device__ __forceinline__ void store_tile(const Params &p, const unsigned char *tile,
                                           const int rows, const int t0, const int c_tile) {
  for (int item = threadIdx.x; item < rows * kChunks; item += kThreads) {
    const int r = item / kChunks, chunk = item % kChunks;
    const int t = t0 + r, c0 = c_tile + chunk * 8;
    if (t < p.length && c0 < p.width)
      *reinterpret_cast<uint4 *>(p.output + static_cast<std::size_t>(t) * p.width + c0) =
          *reinterpret_cast<const uint4 *>(tile + tile_offset(r, chunk));
  }
}

// ------------------------------------------------------------ CUDA cores
// R = outputs per thread and the tap padding unit: 8 for the short filters
// (k <= 8, so k = 7 costs 8 FMAs per output, not 16), 16 otherwise.
template <bool kProj, int TT, int R>
__global__ void __launch_bounds__(kThreads, 2)
gated_fir_simt_kernel(const Params p) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int halo = p.padded_taps - 1;
  unsigned char *const u_tile = smem;
  unsigned char *const x2_tile = u_tile + (TT + halo) * kRowBytes;
  float2 *const h_tile = reinterpret_cast<float2 *>(x2_tile + TT * kRowBytes);  // [delay][pair]
  const int t0 = p.row_begin + blockIdx.x * TT;
  const int c_tile = blockIdx.y * kChannels;
  const int pair = threadIdx.x % 32;
  const int sub = threadIdx.x / 32;
  const int c0 = c_tile + pair * 2;
  const bool channel_ok = c0 < p.width;

  for (int d = sub; d < p.padded_taps; d += kThreads / 32) {
    float2 h = make_float2(0.0F, 0.0F);
    if (channel_ok && d < p.taps) {
      const int tap = p.cross_correlation ? p.taps - 1 - d : d;
      h.x = filter_value(p.filter, p.filter_is_f32,
                         static_cast<std::size_t>(c0 / p.channels_per_group) * p.taps + tap);
      h.y = filter_value(p.filter, p.filter_is_f32,
                         static_cast<std::size_t>((c0 + 1) / p.channels_per_group) * p.taps + tap);
    }
    h_tile[d * 32 + pair] = h;
  }
  build_tiles<kProj>(p, u_tile, x2_tile, reinterpret_cast<unsigned char *>(h_tile + p.padded_taps * 32),
                     TT + halo, t0 - halo, halo, t0, c_tile, blockIdx.x == 0);
  __syncthreads();

  float direct0 = 0.0F, direct1 = 0.0F;
  if (p.direct != nullptr && channel_ok) {
    direct0 = bf2f(p.direct[c0]);
    direct1 = bf2f(p.direct[c0 + 1]);
  }
  for (int pass = 0; pass < TT / (8 * R); ++pass) {
    const int run0 = pass * (8 * R) + sub * R;
    if (t0 + run0 >= p.length) break;
    float acc0[R], acc1[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc0[r] = acc1[r] = 0.0F;
    for (int d0 = p.padded_taps - R; d0 >= 0; d0 -= R) {
      const int base = halo + run0 - d0 - (R - 1);
      float w0[2 * R - 1], w1[2 * R - 1];
#pragma unroll
      for (int i = 0; i < 2 * R - 1; ++i) {
        const std::uint32_t packed = tile_pair(u_tile, base + i, pair);
        w0[i] = lo(packed);
        w1[i] = hi(packed);
      }
#pragma unroll
      for (int dd = R - 1; dd >= 0; --dd) {  // oldest input first
        const float2 h = h_tile[(d0 + dd) * 32 + pair];
#pragma unroll
        for (int r = 0; r < R; ++r) {
          acc0[r] = fmaf(w0[r - dd + R - 1], h.x, acc0[r]);
          acc1[r] = fmaf(w1[r - dd + R - 1], h.y, acc1[r]);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int row = run0 + r;
      float y0 = acc0[r], y1 = acc1[r];
      if (p.direct != nullptr) {
        const std::uint32_t packed = tile_pair(u_tile, halo + row, pair);
        y0 = fmaf(direct0, lo(packed), y0);
        y1 = fmaf(direct1, hi(packed), y1);
      }
      std::uint32_t *const slot = reinterpret_cast<std::uint32_t *>(
          x2_tile + tile_offset(row, pair >> 2) + ((pair & 3) << 2));
      const std::uint32_t gate = *slot;
      *slot = pack_bf16x2(rbf(y0) * lo(gate), rbf(y1) * hi(gate));
    }
  }
  __syncthreads();
  store_tile(p, x2_tile, TT, t0, c_tile);
}

// ---------------------------------------------------------- tensor cores
__device__ __forceinline__ void ldmatrix_x4_trans(const std::uint32_t address,
                                                  std::uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(address));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const std::uint32_t (&a)[4],
                                         const std::uint32_t b0, const std::uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

constexpr int kMmaHalo = 128;  // history rows staged before the tile (>= taps-1, 16-aligned)

// A CTA walks `tiles_per_cta` consecutive TT-row tiles of its 64 channels: only
// the first one builds its 128 history rows from global memory, the later ones
// keep the last 128 rows of u of the tile before (a 16 KB copy inside shared
// memory instead of 128 rows of loads and featurizer work).
template <bool kProj, int TT>
__global__ void __launch_bounds__(kThreads, 2)
gated_fir_mma_kernel(const Params p, const int tiles_per_cta) {
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char *const u_tile = smem;
  unsigned char *const x2_tile = u_tile + (TT + kMmaHalo) * kRowBytes;
  unsigned short *const h_s =
      reinterpret_cast<unsigned short *>(x2_tile + TT * kRowBytes);  // [4 blocks][128] BF16 bits
  const int c_tile = blockIdx.y * kChannels;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int block16 = warp % 4;             // 16-channel block of the tile
  const int part = warp / 4;                // half of the time tile
  const int g = lane / 4, q = lane % 4;

  for (int i = threadIdx.x; i < 4 * 128; i += kThreads) {
    const int block = i / 128, d = i % 128;
    const int channel = c_tile + block * 16;
    unsigned short bits = 0;
    if (channel < p.width && d < p.taps)
      bits = __bfloat16_as_ushort(static_cast<const bf16 *>(
          p.filter)[static_cast<std::size_t>(channel / p.channels_per_group) * p.taps + d]);
    h_s[i] = bits;
  }
  __syncthreads();

  const int channel0 = c_tile + block16 * 16;
  float direct[2][2] = {};
  if (p.direct != nullptr && channel0 < p.width) {
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      direct[nt][0] = bf2f(p.direct[channel0 + 8 * nt + 2 * q]);
      direct[nt][1] = bf2f(p.direct[channel0 + 8 * nt + 2 * q + 1]);
    }
  }
  const std::uint32_t u_base = static_cast<std::uint32_t>(__cvta_generic_to_shared(u_tile));
  unsigned char *const raw = reinterpret_cast<unsigned char *>(h_s + 4 * 128);
  constexpr int kTilesPerWarp = TT / 32;
  static_assert(TT >= kMmaHalo && TT % 8 == 0, "history rows move without overlapping, swizzle unchanged");

  for (int step = 0; step < tiles_per_cta; ++step) {
    const int t0 = p.row_begin + (blockIdx.x * tiles_per_cta + step) * TT;
    if (t0 >= p.length) break;
    if (step > 0) {
      // rows [TT, TT + 128) of the previous tile are this tile's history
      for (int i = threadIdx.x; i < kMmaHalo * kRowBytes / 16; i += kThreads)
        reinterpret_cast<uint4 *>(u_tile)[i] = reinterpret_cast<const uint4 *>(u_tile + TT * kRowBytes)[i];
      __syncthreads();
    }
    // one call site: the first tile also builds its history rows
    const int skip = step == 0 ? 0 : kMmaHalo;
    build_tiles<kProj>(p, u_tile + skip * kRowBytes, x2_tile, raw, TT + kMmaHalo - skip, t0 - kMmaHalo + skip,
                       kMmaHalo - skip, t0, c_tile, step == 0 && blockIdx.x == 0);
    __syncthreads();
    // Toeplitz fragments: H[m][k] = h[128 + m - k] over k in [0, 144).  Rebuilt
    // per tile (27 shared-memory loads) so that they do not occupy registers
    // while the featurizer runs.
    const unsigned short *const h = h_s + block16 * 128;
    auto tap = [&](const int delay) -> std::uint32_t {
      return (delay >= 0 && delay < 128) ? h[delay] : 0U;
    };
    std::uint32_t a_frag[9][4];
#pragma unroll
    for (int j = 0; j < 9; ++j) {
      const int d = 128 + g - (16 * j + 2 * q);  // row g, k = 16j + 2q
      a_frag[j][0] = tap(d) | (tap(d - 1) << 16U);
      a_frag[j][1] = tap(d + 8) | (tap(d + 7) << 16U);
      a_frag[j][2] = tap(d - 8) | (tap(d - 9) << 16U);
      a_frag[j][3] = a_frag[j][0];
    }
    for (int mt = 0; mt < kTilesPerWarp; ++mt) {
      const int row0 = part * (TT / 2) + 16 * mt;  // first output row of this m-tile
      if (t0 + row0 >= p.length) break;
      float acc[2][4] = {};
#pragma unroll
      for (int j = 0; j < 9; ++j) {
        std::uint32_t b[4];
        const int row = row0 + 16 * j + (lane % 8) + ((lane / 8) % 2) * 8;
        ldmatrix_x4_trans(u_base + tile_offset(row, 2 * block16 + lane / 16), b);
        mma_bf16(acc[0], a_frag[j], b[0], b[1]);
        mma_bf16(acc[1], a_frag[j], b[2], b[3]);
      }
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int row = row0 + g + 8 * half;
          const int pair = 8 * block16 + 4 * nt + q;
          float y0 = acc[nt][2 * half], y1 = acc[nt][2 * half + 1];
          if (p.direct != nullptr) {
            const std::uint32_t packed = tile_pair(u_tile, kMmaHalo + row, pair);
            y0 = fmaf(direct[nt][0], lo(packed), y0);
            y1 = fmaf(direct[nt][1], hi(packed), y1);
          }
          std::uint32_t *const slot = reinterpret_cast<std::uint32_t *>(
              x2_tile + tile_offset(row, pair >> 2) + ((pair & 3) << 2));
          const std::uint32_t gate = *slot;
          *slot = pack_bf16x2(rbf(y0) * lo(gate), rbf(y1) * hi(gate));
        }
    }
    __syncthreads();
    store_tile(p, x2_tile, TT, t0, c_tile);
    __syncthreads();  // both tiles are rewritten by the next step
  }
}

// ------------------------------------------------------- register streaming
// Short filters (k <= 8): no shared memory at all.  A thread owns four
// neighbouring channels and walks down a segment of rows; the 3-tap featurizer
// history (two raw rows) and the last k-1 values of u live in registers, so
// every input element is loaded exactly once per segment (plus k+1 warm-up rows
// per segment) with 8-byte loads, and the loads of the next kUnroll rows are in
// flight while the current ones are computed.  Same FMA order and rounding
// points as the tiled kernel above.
constexpr int kStreamThreads = 128;

// kC/2 packed pairs from 4-byte-aligned (kC = 2) or 8-byte-aligned (kC = 4) memory
template <int kC>
__device__ __forceinline__ void load_pairs(const bf16 *source, std::uint32_t *words) {
  if constexpr (kC == 4) {
    const uint2 v = __ldcs(reinterpret_cast<const uint2 *>(source));
    words[0] = v.x;
    words[1] = v.y;
  } else {
    words[0] = __ldcs(reinterpret_cast<const unsigned int *>(source));
  }
}
template <int kC>
__device__ __forceinline__ void store_pairs(bf16 *target, const std::uint32_t *words) {
  if constexpr (kC == 4)
    *reinterpret_cast<uint2 *>(target) = make_uint2(words[0], words[1]);
  else
    *reinterpret_cast<unsigned int *>(target) = words[0];
}

// Product of two packed BF16 pairs, each rounded once: the same bits as
// widening, multiplying in F32 (exact for BF16 operands) and rounding back.
__device__ __forceinline__ std::uint32_t mul_pairs(const std::uint32_t a, const std::uint32_t b) {
  std::uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

template <bool kProj, int kTaps, int kC, int kUnroll, int kResident>
__global__ void __launch_bounds__(kStreamThreads, kResident)
gated_fir_stream_kernel(const Params p, const int segment_rows) {
  constexpr int kHalo = kTaps - 1;
  constexpr int kWarm = ((kProj ? kHalo + 2 : kHalo) + kUnroll - 1) / kUnroll * kUnroll;
  constexpr int kPairs = kC / 2;
  constexpr int kWords = 3 * kPairs;  // words of one row: 3 kC raw columns, or x1 | v | x2
  const int c0 = (blockIdx.x * kStreamThreads + threadIdx.x) * kC;
  if (c0 >= p.width) return;
  const int t_own = p.row_begin + blockIdx.y * segment_rows;
  const int t_end = min(p.length, t_own + segment_rows);
  if (t_own >= t_end) return;

  // h[d] multiplies u[t - d]; taps beyond the filter are zero
  float h[kTaps];
  {
    const std::size_t base = static_cast<std::size_t>(c0 / p.channels_per_group) * p.taps;
#pragma unroll
    for (int d = 0; d < kTaps; ++d)
      h[d] = d < p.taps ? filter_value(p.filter, p.filter_is_f32,
                                       base + (p.cross_correlation ? p.taps - 1 - d : d))
                        : 0.0F;
  }
  const bool has_direct = p.direct != nullptr;
  float direct[kC];
#pragma unroll
  for (int c = 0; c < kC; ++c) direct[c] = has_direct ? bf2f(p.direct[c0 + c]) : 0.0F;
  // featurizer taps of the 3 kC columns, [column][tap] as stored
  float st[kProj ? 3 * kC : 1][3];
  if constexpr (kProj) {
    const unsigned int *const source =
        reinterpret_cast<const unsigned int *>(p.short_filter + static_cast<std::size_t>(c0) * 9);
#pragma unroll
    for (int i = 0; i < 9 * kPairs; ++i) {
      const unsigned int w = __ldg(source + i);
      st[(2 * i) / 3][(2 * i) % 3] = lo(w);
      st[(2 * i + 1) / 3][(2 * i + 1) % 3] = hi(w);
    }
  }

  struct Row {
    std::uint32_t w[kWords];
  };
  // kChecked: the row may lie before the sequence, before this segment (no x2
  // needed) or behind its end
  const auto load_row = [&](auto checked, const int t) {
    constexpr bool kChecked = decltype(checked)::value;
    Row row;
    if constexpr (kChecked) {
#pragma unroll
      for (int i = 0; i < kWords; ++i) row.w[i] = 0U;
      if (t < 0 || t >= t_end) return row;
    }
    if constexpr (kProj) {
      const bf16 *const source =
          p.projection + static_cast<std::size_t>(t) * 3 * p.width + static_cast<std::size_t>(c0) * 3;
#pragma unroll
      for (int i = 0; i < 3; ++i) load_pairs<kC>(source + i * kC, row.w + i * kPairs);
    } else {
      const std::size_t index = static_cast<std::size_t>(t) * p.width + c0;
      load_pairs<kC>(p.x1 + index, row.w);
      load_pairs<kC>(p.value + index, row.w + kPairs);
      if (!kChecked || t >= t_own) load_pairs<kC>(p.x2 + index, row.w + 2 * kPairs);
    }
    return row;
  };
  // The rows are loaded in order, one call per row from the first warm-up row on: the
  // projection-fed form carries the row's address along instead of rebuilding it from t.
  [[maybe_unused]] std::intptr_t cursor =
      reinterpret_cast<std::intptr_t>(p.projection) +
      (static_cast<std::intptr_t>(t_own - kWarm) * 3 * p.width + static_cast<std::intptr_t>(c0) * 3) *
          static_cast<std::intptr_t>(sizeof(bf16));
  [[maybe_unused]] const std::intptr_t cursor_stride = static_cast<std::intptr_t>(p.width) * 3 * sizeof(bf16);
  const auto load_next_row = [&](auto checked, const int t) {
    if constexpr (!kProj) {
      return load_row(checked, t);
    } else {
      constexpr bool kChecked = decltype(checked)::value;
      Row row;
      const bf16 *const source = reinterpret_cast<const bf16 *>(cursor);
      cursor += cursor_stride;
      if constexpr (kChecked) {
#pragma unroll
        for (int i = 0; i < kWords; ++i) row.w[i] = 0U;
        if (t < 0 || t >= t_end) return row;
      }
#pragma unroll
      for (int i = 0; i < 3; ++i) load_pairs<kC>(source + i * kC, row.w + i * kPairs);
      return row;
    }
  };

  float xh[2][kProj ? 3 * kC : 1];   // raw rows t-2, t-1
#pragma unroll
  for (int i = 0; i < (kProj ? 3 * kC : 1); ++i) xh[0][i] = xh[1][i] = 0.0F;
  float uw[kHalo > 0 ? kHalo : 1][kC];  // uw[d - 1] = u[t - d]
#pragma unroll
  for (int d = 0; d < (kHalo > 0 ? kHalo : 1); ++d)
#pragma unroll
    for (int c = 0; c < kC; ++c) uw[d][c] = 0.0F;
  const int real_halo = p.taps - 1;
  // first row whose u belongs to the decode history
  const int cache_begin = (p.inner_cache != nullptr && real_halo > 0) ? p.length - real_halo : p.length;
  const int t_first = t_own - kWarm;

  Row next[kUnroll];
  std::size_t out_offset = static_cast<std::size_t>(t_own) * p.width + c0;
  const auto run_group = [&](auto checked, const int base) {
    constexpr bool kChecked = decltype(checked)::value;
    Row rows[kUnroll];
#pragma unroll
    for (int i = 0; i < kUnroll; ++i) rows[i] = next[i];
#pragma unroll
    for (int i = 0; i < kUnroll; ++i) next[i] = load_next_row(checked, base + kUnroll + i);
#pragma unroll
    for (int i = 0; i < kUnroll; ++i) {
      const int t = base + i;
      std::uint32_t u_pair[kPairs], gate_pair[kPairs];
      if constexpr (kProj) {
        float z[3 * kC];
#pragma unroll
        for (int w = 0; w < kWords; ++w) {
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int column = 2 * w + half;
            const float x = half == 0 ? lo(rows[i].w[w]) : hi(rows[i].w[w]);
            // fmaf with +0, not a multiply: the sign of a zero result must match the FMA chain
            float acc = fmaf(xh[0][column], st[column][0], 0.0F);
            acc = fmaf(xh[1][column], st[column][1], acc);
            z[column] = fmaf(x, st[column][2], acc);
            xh[0][column] = xh[1][column];
            xh[1][column] = x;
          }
        }
#pragma unroll
        for (int j = 0; j < kPairs; ++j) {
          const int a = 6 * j, b = 6 * j + 3;  // first columns (x2, x1, v) of the two channels
          gate_pair[j] = round_pair_bf16(z[a], z[b]);
          u_pair[j] = mul_pairs(round_pair_bf16(z[a + 1], z[b + 1]), round_pair_bf16(z[a + 2], z[b + 2]));
        }
      } else {
#pragma unroll
        for (int j = 0; j < kPairs; ++j) {
          u_pair[j] = mul_pairs(rows[i].w[j], rows[i].w[kPairs + j]);
          gate_pair[j] = rows[i].w[2 * kPairs + j];
        }
      }
      float u[kC];
#pragma unroll
      for (int j = 0; j < kPairs; ++j) {
        u[2 * j] = lo(u_pair[j]);
        u[2 * j + 1] = hi(u_pair[j]);
      }
      if (!kChecked || (t >= t_own && t < t_end)) {
        float y[kC];
#pragma unroll
        for (int c = 0; c < kC; ++c) {
          float acc = 0.0F;
#pragma unroll
          for (int d = kHalo; d >= 1; --d) acc = fmaf(uw[d - 1][c], h[d], acc);  // oldest input first
          acc = fmaf(u[c], h[0], acc);
          if (has_direct) acc = fmaf(direct[c], u[c], acc);
          y[c] = acc;
        }
        std::uint32_t packed[kPairs];
#pragma unroll
        for (int j = 0; j < kPairs; ++j)
          packed[j] = mul_pairs(round_pair_bf16(y[2 * j], y[2 * j + 1]), gate_pair[j]);
        // rows t_own .. t_end - 1 come by in order: the offset t * width + c0 is carried along
        store_pairs<kC>(p.output + out_offset, packed);
        if (p.pregate != nullptr) store_pairs<kC>(p.pregate + out_offset, u_pair);
        out_offset += static_cast<std::size_t>(p.width);
      }
      if constexpr (kChecked && kProj) {
        // raw rows length-2 and length-1 are the featurizer's decode history
        if (p.short_cache != nullptr && t == p.length - 1) {
#pragma unroll
          for (int column = 0; column < 3 * kC; ++column)
            *reinterpret_cast<float2 *>(p.short_cache + (static_cast<std::size_t>(c0) * 3 + column) * 2) =
                make_float2(xh[0][column], xh[1][column]);
        }
      }
      if constexpr (kChecked) {
        // The first segment of a row window also owns the history rows it
        // recomputes, so that the decode history is complete even for windows
        // shorter than it.
        if (t >= cache_begin && t < t_end &&
            (t >= t_own || (blockIdx.y == 0 && t >= 0 && t >= t_own - kHalo))) {
          const int slot = t - cache_begin;
#pragma unroll
          for (int c = 0; c < kC; ++c) p.inner_cache[static_cast<std::size_t>(c0 + c) * real_halo + slot] = u[c];
        }
      }
#pragma unroll
      for (int d = kHalo - 1; d >= 1; --d)
#pragma unroll
        for (int c = 0; c < kC; ++c) uw[d][c] = uw[d - 1][c];
      if constexpr (kHalo > 0) {
#pragma unroll
        for (int c = 0; c < kC; ++c) uw[0][c] = u[c];
      }
    }
  };

  constexpr std::true_type kCheckedRows{};
  constexpr std::false_type kPlainRows{};
#pragma unroll
  for (int i = 0; i < kUnroll; ++i) next[i] = load_next_row(kCheckedRows, t_first + i);
  int base = t_first;
  for (; base < t_own; base += kUnroll) run_group(kCheckedRows, base);  // warm-up: kWarm is a multiple of kUnroll
  // steady state: this group and the one being fetched lie inside the segment,
  // in front of the rows that feed the decode history
  const int plain_end = min(t_end, cache_begin);
  for (; base + 2 * kUnroll <= plain_end; base += kUnroll) run_group(kPlainRows, base);
  for (; base < t_end; base += kUnroll) run_group(kCheckedRows, base);
}

template <bool kProj, int kTaps, int kC, int kUnroll, int kResident>
int launch_stream(const Params &p, cudaStream_t stream) {
  const auto kernel = gated_fir_stream_kernel<kProj, kTaps, kC, kUnroll, kResident>;
  static const int resident = [&] {
    int blocks = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, kernel, kStreamThreads, 0) != cudaSuccess ||
        blocks < 1)
      blocks = 1;
    return blocks;
  }();
  // One wave of CTAs: as many row segments as fill every SM once, none shorter
  // than 32 rows (each segment recomputes k+1 warm-up rows).
  const int rows = p.length - p.row_begin;
  const int across = static_cast<int>(ceil_div_u(p.width, kStreamThreads * kC));
  int segments = std::max(1, kSmCount * resident / across);
  segments = std::max(1, std::min(segments, rows / 32));
  const int segment_rows = (rows + segments - 1) / segments;
  const dim3 grid(across, ceil_div_u(rows, segment_rows));
  kernel<<<grid, kStreamThreads, 0, stream>>>(p, segment_rows);
  return check_launch("streaming FIR kernel");
}

template <bool kProj>
int launch_stream_taps(const Params &p, cudaStream_t stream) {
  // k = 7 is the shape of every released model; other short filters pad to 8.
  // Four channels per thread with four rows of loads in flight measured best
  // (against two channels, or eight rows).
  // The projection-fed form needs ~200 registers: two resident CTAs without
  // spills measured faster than three with.
  if (p.taps == 7) return launch_stream<kProj, 7, 4, 4, kProj ? 2 : 4>(p, stream);
  return launch_stream<kProj, 8, 4, 4, kProj ? 2 : 4>(p, stream);
}

template <typename Kernel>
int launch(Kernel kernel, const Params &p, const int tile_rows, const std::size_t smem,
           cudaStream_t stream, const char *what) {
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(smem)) != cudaSuccess)
    return fail(kCuda, "cannot raise the fused FIR shared-memory limit");
  const dim3 grid(ceil_div_u(p.length - p.row_begin, tile_rows), ceil_div_u(p.width, kChannels));
  if (grid.y > 65535) return fail(kInvalidArgument, "gated FIR is too wide");
  kernel<<<grid, kThreads, smem, stream>>>(p);
  return check_launch(what);
}

// Grid of the Toeplitz kernel: each CTA walks as many consecutive tiles as it
// takes for the grid to fit the resident slots once ...
template <bool kProj, int TT>
int launch_mma(const Params &p, const std::size_t smem, cudaStream_t stream) {
  const auto kernel = gated_fir_mma_kernel<kProj, TT>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) !=
      cudaSuccess)
    return fail(kCuda, "cannot raise the fused FIR shared-memory limit");
  static const int resident = [&] {
    int blocks = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, kernel, kThreads, smem) != cudaSuccess || blocks < 1)
      blocks = 1;
    return blocks;
  }();
  const unsigned int tiles = ceil_div_u(p.length - p.row_begin, TT);
  const unsigned int across = ceil_div_u(p.width, kChannels);
  if (across > 65535) return fail(kInvalidArgument, "gated FIR is too wide");
  const unsigned int slots = static_cast<unsigned int>(kSmCount * resident);
  const unsigned int segments = std::max(1U, std::min(tiles, slots / std::max(1U, across)));
  // ... but no more than 8 tiles each: longer walks keep the two CTAs of an SM in
  // the same phase (both loading, then both on the tensor cores) and measured slower.
  const int tiles_per_cta = std::min(8, static_cast<int>(ceil_div_u(tiles, segments)));
  const dim3 grid(ceil_div_u(tiles, tiles_per_cta), across);
  kernel<<<grid, kThreads, smem, stream>>>(p, tiles_per_cta);
  return check_launch("fused Toeplitz FIR kernel");
}

bool aligned16(const void *ptr) { return (reinterpret_cast<std::uintptr_t>(ptr) & 15U) == 0; }

}  // namespace

int gated_fir_prefill(const GatedFirArgs &a, cudaStream_t stream) {
  const bool from_projection = a.projection != nullptr;
  const bool inputs_ok =
      from_projection ? (a.short_filter != nullptr && a.short_taps == 3 && aligned16(a.projection) &&
                         aligned16(a.short_filter))
                      : (a.x2 != nullptr && a.x1 != nullptr && a.value != nullptr && aligned16(a.x2) &&
                         aligned16(a.x1) && aligned16(a.value));
  if (!inputs_ok || a.filter == nullptr || a.output == nullptr || a.width == 0 || a.groups == 0 ||
      a.width % 8 != 0 || a.width % a.groups != 0 || a.taps == 0 || a.taps > 128 ||
      a.length == 0 || a.row_begin >= a.length || a.length > 0x7fff0000U || !aligned16(a.output) ||
      (a.pregate != nullptr && !aligned16(a.pregate)))
    return gated_fir_prefill_generic(a, stream);  // validates and reports
  // the streaming kernel writes every history slot that has a row and the
  // featurizer history itself
  const bool streaming = a.taps <= 8 && (a.width / a.groups) % 4 == 0;
  if (a.inner_cache != nullptr && a.taps > 1 && (!streaming || a.length < a.taps - 1) &&
      cudaMemsetAsync(a.inner_cache, 0, a.width * (a.taps - 1) * sizeof(float), stream) != cudaSuccess)
    return fail(kCuda, "cannot clear the FIR cache");
  Params p{};
  p.x2 = static_cast<const bf16 *>(a.x2);
  p.x1 = static_cast<const bf16 *>(a.x1);
  p.value = static_cast<const bf16 *>(a.value);
  p.projection = static_cast<const bf16 *>(a.projection);
  p.short_filter = static_cast<const bf16 *>(a.short_filter);
  p.direct = static_cast<const bf16 *>(a.direct);
  p.filter = a.filter;
  p.output = static_cast<bf16 *>(a.output);
  p.pregate = static_cast<bf16 *>(a.pregate);
  p.inner_cache = a.inner_cache;
  p.length = static_cast<int>(a.length);
  p.row_begin = static_cast<int>(a.row_begin);
  p.width = static_cast<int>(a.width);
  p.taps = static_cast<int>(a.taps);
  const std::size_t run = a.taps <= 8 ? 8 : kRun;
  p.padded_taps = static_cast<int>((a.taps + run - 1) / run * run);
  p.channels_per_group = static_cast<int>(a.width / a.groups);
  p.filter_is_f32 = a.filter_is_f32;
  p.cross_correlation = a.cross_correlation;
  int status;
  const bool tensor = !a.cross_correlation && !a.filter_is_f32 && a.taps > 32 &&
                      p.channels_per_group % 16 == 0;
  static const bool tcgen05_off = [] {
    const char *const flag = std::getenv("EVO_B200_HCM_TCGEN05");
    return flag != nullptr && flag[0] == '0';
  }();
  if (tensor && !tcgen05_off && gated_fir_tcgen05_applicable(a)) {
    status = gated_fir_tcgen05(a, stream);
  } else if (tensor) {
    constexpr int TT = 256;
    const std::size_t smem = (TT + kMmaHalo) * kRowBytes + TT * kRowBytes + 4 * 128 * 2 +
                             (from_projection ? kRawBytes : 0);
    status = from_projection ? launch_mma<true, TT>(p, smem, stream) : launch_mma<false, TT>(p, smem, stream);
  } else if (streaming) {
    p.short_cache = from_projection && a.short_taps == 3 ? a.short_cache : nullptr;
    status = from_projection ? launch_stream_taps<true>(p, stream) : launch_stream_taps<false>(p, stream);
  } else if (p.padded_taps <= 8) {
    constexpr int TT = 256;
    const std::size_t smem = (TT + p.padded_taps - 1) * kRowBytes + TT * kRowBytes +
                             static_cast<std::size_t>(p.padded_taps) * 32 * sizeof(float2) +
                             (from_projection ? kRawBytes : 0);
    status = from_projection
                 ? launch(gated_fir_simt_kernel<true, TT, 8>, p, TT, smem, stream, "fused FIR kernel")
                 : launch(gated_fir_simt_kernel<false, TT, 8>, p, TT, smem, stream, "fused FIR kernel");
  } else if (p.padded_taps <= 32) {
    constexpr int TT = 256;
    const std::size_t smem = (TT + p.padded_taps - 1) * kRowBytes + TT * kRowBytes +
                             static_cast<std::size_t>(p.padded_taps) * 32 * sizeof(float2) +
                             (from_projection ? kRawBytes : 0);
    status = from_projection
                 ? launch(gated_fir_simt_kernel<true, TT, 16>, p, TT, smem, stream, "fused FIR kernel")
                 : launch(gated_fir_simt_kernel<false, TT, 16>, p, TT, smem, stream, "fused FIR kernel");
  } else {
    constexpr int TT = 128;
    const std::size_t smem = (TT + p.padded_taps - 1) * kRowBytes + TT * kRowBytes +
                             static_cast<std::size_t>(p.padded_taps) * 32 * sizeof(float2) +
                             (from_projection ? kRawBytes : 0);
    status = from_projection
                 ? launch(gated_fir_simt_kernel<true, TT, 16>, p, TT, smem, stream, "fused FIR kernel")
                 : launch(gated_fir_simt_kernel<false, TT, 16>, p, TT, smem, stream, "fused FIR kernel");
  }
  if (status != kOk) return status;
  if (a.short_cache != nullptr && from_projection && a.short_taps > 1 && p.short_cache == nullptr)
    status = fill_fir_cache(a.projection, a.short_cache, a.length, a.width * 3, a.short_taps - 1, stream);
  return status;
}

}  // namespace evob
