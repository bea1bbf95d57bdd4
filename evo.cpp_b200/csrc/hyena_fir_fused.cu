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
                                            const int t_own, const int c_tile) {
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
    const bool owns = t >= t_own || (blockIdx.x == 0 && t >= 0);
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
                     TT + halo, t0 - halo, halo, t0, c_tile);
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

template <bool kProj, int TT>
__global__ void __launch_bounds__(kThreads, 2)
gated_fir_mma_kernel(const Params p) {
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char *const u_tile = smem;
  unsigned char *const x2_tile = u_tile + (TT + kMmaHalo) * kRowBytes;
  unsigned short *const h_s =
      reinterpret_cast<unsigned short *>(x2_tile + TT * kRowBytes);  // [4 blocks][128] BF16 bits
  const int t0 = p.row_begin + blockIdx.x * TT;
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
  build_tiles<kProj>(p, u_tile, x2_tile, reinterpret_cast<unsigned char *>(h_s + 4 * 128),
                     TT + kMmaHalo, t0 - kMmaHalo, kMmaHalo, t0, c_tile);
  __syncthreads();

  // Toeplitz fragments: H[m][k] = h[128 + m - k] over k in [0, 144).
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
  constexpr int kTilesPerWarp = TT / 32;
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
  if (a.inner_cache != nullptr && a.taps > 1 &&
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
  if (tensor) {
    constexpr int TT = 256;
    const std::size_t smem = (TT + kMmaHalo) * kRowBytes + TT * kRowBytes + 4 * 128 * 2 +
                             (from_projection ? kRawBytes : 0);
    status = from_projection
                 ? launch(gated_fir_mma_kernel<true, TT>, p, TT, smem, stream, "fused Toeplitz FIR kernel")
                 : launch(gated_fir_mma_kernel<false, TT>, p, TT, smem, stream, "fused Toeplitz FIR kernel");
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
  if (a.short_cache != nullptr && from_projection && a.short_taps > 1)
    status = fill_fir_cache(a.projection, a.short_cache, a.length, a.width * 3, a.short_taps - 1, stream);
  return status;
}

}  // namespace evob
