// Medium-regularised Hyena operator (HCM, k <= 128) on the 5th-generation
// tensor cores, fed by the raw interleaved projection:
//   u = bf16(x1 * v),  y = bf16(sum_k h[g,k] u[t-k] + D u),  out = bf16(y * x2)
// with (x2, x1, v) the 3-tap featurizer of the projection's channel triples
// (upstream: short FIR, split, gate, FFT convolution, post-gate as separate
// passes, src/cuda/model.cu:1431-1520 and src/cuda/hyena.cu:418-519, 1874-1992).
//
// A group of 16 channels shares one filter, so for 128 consecutive rows the
// convolution is a GEMM  Y[128 x 16] = H[128 x 256] . U[256 x 16]  with the
// banded Toeplitz matrix H[m][k] = h[m + 128 - k] over the 256 rows of u that
// end with the tile.  One CTA owns a group and walks a range of row tiles:
//   warps 0-7  stage the group's 96-byte projection rows two tiles ahead (cp.async
//              reporting to an mbarrier) and build u: a thread owns a channel pair and four
//              consecutive rows, keeps its 18 featurizer taps in registers as F32
//              and unpacks a raw value once for the three rows that use it
//              (rounding points of the unfused chain); u goes out as the K-major
//              swizzled B operand [16 channels x time] into a ring of 64-row K
//              blocks, the x2 gate beside it.  Two iterations later the same
//              warps turn the tile's accumulator into outputs: tcgen05.ld (a
//              row is a TMEM lane), direct term, round, gate, one 16-byte store.
//   warp 8     one lane issues tcgen05.mma M128 N16 K16, sixteen per tile, into
//              one of two 16-column TMEM accumulators; a tile's MMAs run under
//              the featurizer of the tile after it.
// Every hand-over is an mbarrier; there is no CTA-wide barrier in the loop, so
// the warps of a CTA drift apart and fill each other's latencies.
// H depends on the group only and is Toeplitz, so its four 64-column K blocks
// are row windows, 64 rows apart, of one strip T[r][j] = h[r - j] of 320 rows
// (40 KiB instead of 64): the A descriptors just start at different rows.
// The last 128 rows of u of a tile are the first two K blocks of the next one,
// so nothing is recomputed inside a CTA's range; a range starts by building the
// 128 rows in front of it.  Every wait is time-bounded and raises the sticky
// error word of the projection kernels.
#include <cuda.h>

#include <algorithm>

#include "common.cuh"
#include "ops_internal.hpp"
#include "projection_featurizer.cuh"  // round_pair_bf16
#include "tcgen05.cuh"

namespace evob {
namespace {
using namespace tc;

constexpr int kTile = 128;                    // rows per MMA tile
constexpr int kGroup = 16;                    // channels per filter group = N
constexpr int kWorkers = 256;                 // producer / epilogue threads (warps 0-7)
constexpr int kThreadsTotal = kWorkers + 32;  // + the MMA warp
constexpr int kMmaWarp = kWorkers / 32;
constexpr int kStripRows = 320;               // T[r - 64 .. r + 255]
constexpr int kStripBytes = kStripRows * 128;
constexpr int kBlockBytes = kGroup * 128;     // one K block of B: 16 channel rows x 64 time steps
constexpr int kRingBlocks = 6;
constexpr int kRawStride = 112;               // row pitch in shared memory: rows four apart land 16 banks apart
constexpr int kRawRows = kTile + 2;
constexpr int kRawBytes = kRawRows * kRawStride;
constexpr int kRawBuffers = 3;

constexpr int kStripOffset = 0;
constexpr int kRingOffset = kStripOffset + kStripBytes;
constexpr int kRawOffset = kRingOffset + kRingBlocks * kBlockBytes;
constexpr int kGateOffset = kRawOffset + kRawBuffers * kRawBytes;     // [channel][time] gate, three steps x two K blocks
constexpr int kFilterOffset = kGateOffset + 6 * kBlockBytes;          // 128 + 8 BF16 taps
constexpr int kBarrierOffset = kFilterOffset + 1024;
constexpr int kBarriers = 14;  // b_full[2], acc_full[2], acc_empty[2], raw_full[3], raw_empty[3], step_done[2]
constexpr int kTmemPtrOffset = kBarrierOffset + kBarriers * 8;
constexpr int kAbortOffset = kTmemPtrOffset + 8;
constexpr int kSmemBytes = kAbortOffset + 8 + 1024;  // + alignment slack
static_assert(kRawBytes % 16 == 0 && kRingOffset % 1024 == 0 && kFilterOffset % 16 == 0, "tiles keep their alignment");

struct TcParams {
  const bf16 *projection, *short_filter, *filter, *direct;
  bf16 *output, *pregate;
  float *inner_cache;
  int length, row_begin, width, taps, tiles_per_cta;
};

__host__ __device__ constexpr std::uint32_t fir_instruction_descriptor() {
  std::uint32_t d = 0;
  d |= 1U << 4U;   // accumulator F32
  d |= 1U << 7U;   // A BF16
  d |= 1U << 10U;  // B BF16, both K-major
  d |= static_cast<std::uint32_t>(kGroup >> 3) << 17U;
  d |= static_cast<std::uint32_t>(kTile >> 4) << 24U;
  return d;
}

__device__ __forceinline__ void tmem_load_8(const std::uint32_t taddr, std::uint32_t (&v)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
               : "r"(taddr)
               : "memory");
}

__global__ void __launch_bounds__(kThreadsTotal, 2)
gated_fir_tcgen05_kernel(const TcParams p, int *const error_word) {
  extern __shared__ unsigned char smem_raw[];
  // aligned by pointer arithmetic, not through an integer: the compiler keeps the shared address space
  // and every access below is a 32-bit shared load or store rather than a generic one
  unsigned char *const smem = smem_raw + ((1024U - (smem_u32(smem_raw) & 1023U)) & 1023U);
  const std::uint32_t smem_base = smem_u32(smem);
  auto bar = [&](const int index) { return smem_base + kBarrierOffset + 8U * index; };
  enum { kBFull = 0, kAccFull = 2, kAccEmpty = 4, kRawFull = 6, kRawEmpty = 9, kStepDone = 12 };
  volatile std::uint32_t *const tmem_ptr = reinterpret_cast<volatile std::uint32_t *>(smem + kTmemPtrOffset);
  volatile int *const abort_flag = reinterpret_cast<volatile int *>(smem + kAbortOffset);
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int group = blockIdx.y;
  const int c0 = group * kGroup;
  // this CTA's rows: tiles [first_tile, first_tile + tiles) of the rows from row_begin on
  const int all_tiles = (p.length - p.row_begin + kTile - 1) / kTile;
  const int first_tile = blockIdx.x * p.tiles_per_cta;
  const int tiles = min(p.tiles_per_cta, all_tiles - first_tile);
  const int t_first = p.row_begin + first_tile * kTile;  // first output row of the range

  if (threadIdx.x == 0) {
    mbar_init(bar(kBFull), kWorkers);
    mbar_init(bar(kBFull + 1), kWorkers);
    mbar_init(bar(kAccFull), 1);
    mbar_init(bar(kAccFull + 1), 1);
    mbar_init(bar(kAccEmpty), kWorkers);
    mbar_init(bar(kAccEmpty + 1), kWorkers);
    for (int b = 0; b < kRawBuffers; ++b) {
      mbar_init(bar(kRawFull + b), kWorkers);
      mbar_init(bar(kRawEmpty + b), kWorkers);
    }
    mbar_init(bar(kStepDone), kWorkers);
    mbar_init(bar(kStepDone + 1), kWorkers);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(const_cast<std::uint32_t *>(tmem_ptr))),
                 "r"(32U)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // filter taps and the Toeplitz strip (workers), while the MMA warp allocates
  bf16 *const taps_smem = reinterpret_cast<bf16 *>(smem + kFilterOffset);  // [136], zero past `taps`
  if (threadIdx.x < 136)
    taps_smem[threadIdx.x] = threadIdx.x < p.taps ? p.filter[static_cast<std::size_t>(group) * p.taps + threadIdx.x]
                                                  : __ushort_as_bfloat16(0);
  __syncthreads();
  if (warp < kMmaWarp) {
    // T[rho][j] = h[rho - 64 - j]; 16-byte chunks of 8 columns, swizzled like a K-major tile
    for (int chunk = threadIdx.x; chunk < kStripRows * 8; chunk += kWorkers) {
      const int rho = chunk / 8, q = chunk % 8;
      std::uint32_t words[4];
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        unsigned int pair = 0U;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int index = rho - 64 - (8 * q + 2 * w + e);
          const unsigned int bits =
              index >= 0 && index < 128 ? __bfloat16_as_ushort(taps_smem[index]) : 0U;
          pair |= bits << (16 * e);
        }
        words[w] = pair;
      }
      *reinterpret_cast<uint4 *>(smem + kStripOffset + rho * 128 + ((q ^ (rho & 7)) << 4)) =
          make_uint4(words[0], words[1], words[2], words[3]);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const std::uint32_t tmem_base = *tmem_ptr;

  if (warp == kMmaWarp) {
    if (lane == 0 && tiles > 0) {
      constexpr std::uint32_t idesc = fir_instruction_descriptor();
      // production step s writes K blocks 2s, 2s + 1 (step 0 = the 128 rows in front of the range);
      // tile i needs steps i and i + 1, i.e. K blocks 2i .. 2i + 3
      for (int i = 0; i < tiles; ++i) {
        const int step = i + 1;
        if (!mbar_wait(bar(kBFull + (step & 1)), (step >> 1) & 1U, abort_flag)) break;
        if (i == 0 && !mbar_wait(bar(kBFull), 0U, abort_flag)) break;  // step 0
        const int acc = i & 1;
        if (!mbar_wait(bar(kAccEmpty + acc), ((i >> 1) & 1U) ^ 1U, abort_flag)) break;
        tc_fence_after();
#pragma unroll
        for (int kb = 0; kb < 4; ++kb) {
          const std::uint32_t a_base = smem_base + kStripOffset + (192 - 64 * kb) * 128;
          const std::uint32_t b_base = smem_base + kRingOffset + ((2 * i + kb) % kRingBlocks) * kBlockBytes;
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc_mma<false>(tmem_base + acc * kGroup, smem_descriptor(a_base) + 2U * k, smem_descriptor(b_base) + 2U * k,
                          idesc, (kb | k) != 0 ? 1U : 0U);
        }
        tc_commit(bar(kAccFull + acc));
      }
    }
  } else {
    // ------------------------------------------------------------ workers
    // Production: thread = (channel pair cp of the group, four consecutive rows 4 * quad ..).  Its 18
    // featurizer taps sit in registers as F32, and a raw value that three neighbouring rows use is
    // unpacked once.  Epilogue: thread = (row of the tile, half of the channels), its row being
    // a TMEM lane; u and the gate come back from shared memory, both kept [channel][time].
    // Warps run free: every hand-over is an mbarrier, none a CTA-wide barrier.
    const int cp = threadIdx.x % 8, quad = threadIdx.x / 8;
    const int row = threadIdx.x % kTile, half = threadIdx.x / kTile;
    // taps[column][k]: columns (x2, x1, v) of channel 2cp, then of channel 2cp + 1; k oldest first
    float taps[6][3];
    {
      const std::uint32_t *const packed =
          reinterpret_cast<const std::uint32_t *>(p.short_filter + static_cast<std::size_t>(c0 + 2 * cp) * 9);
#pragma unroll
      for (int w = 0; w < 9; ++w) {
        const std::uint32_t word = __ldg(packed + w);
        taps[(2 * w) / 3][(2 * w) % 3] = __uint_as_float(word << 16U);
        taps[(2 * w + 1) / 3][(2 * w + 1) % 3] = __uint_as_float(word & 0xffff0000U);
      }
    }
    float direct[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) direct[c] = p.direct != nullptr ? bf2f(p.direct[c0 + half * 8 + c]) : 0.0F;
    // Raw rows [t0 - 2, t0 + 128) of the group's columns, 780 copies of 16 bytes (zero-filled
    // outside [0, length)): a thread's (row, chunk) assignments do not change from step to step,
    // and its copies report to the buffer's mbarrier when they land.
    const unsigned char *const group_columns =
        reinterpret_cast<const unsigned char *>(p.projection + static_cast<std::size_t>(c0) * 3);
    const std::size_t row_bytes = static_cast<std::size_t>(p.width) * 6;
    int stage_row[4], stage_smem[4], stage_global[4];
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const int item = threadIdx.x + n * kWorkers;
      stage_row[n] = item / 6 - 2;  // relative to t0
      stage_smem[n] = (item / 6) * kRawStride + (item % 6) * 16;
      stage_global[n] = (item / 6 - 2) * p.width * 6 + (item % 6) * 16;  // bytes from row t0
    }
    const auto stage_raw = [&](const int step) {
      const int t0 = t_first + (step - 1) * kTile;
      const int buffer = step % kRawBuffers;
      const std::uint32_t base = smem_base + kRawOffset + buffer * kRawBytes;
      const unsigned char *const origin = group_columns + static_cast<std::ptrdiff_t>(t0) * static_cast<std::ptrdiff_t>(row_bytes);
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        if (n == 3 && threadIdx.x + 3 * kWorkers >= kRawRows * 6) break;
        const int t = t0 + stage_row[n];
        // The oldest raw row of step 0 only feeds u[t_first - 128], which meets a zero tap: it is not
        // read, so a window needs taps + 1 = 129 rows of history in front of it, as the other kernels do.
        const bool valid = t >= 0 && t < p.length && (step != 0 || stage_row[n] != -2);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(base + stage_smem[n]),
                     "l"(valid ? origin + stage_global[n] : reinterpret_cast<const unsigned char *>(p.projection)),
                     "r"(valid ? 16U : 0U)
                     : "memory");
      }
      asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar(kRawFull + buffer)) : "memory");
    };
    if (tiles > 0) {
      stage_raw(0);
      stage_raw(1);
    }

    // production step s covers rows [t_first + (s - 1) * 128, + 128): step 0 is the history in
    // front of the range, step s >= 1 the rows of tile s - 1.  Tile i is multiplied once step
    // i + 1 is published and turned into outputs in iteration i + 2, so the tensor core works
    // under the next step's featurizer.  Iteration s = production of step s, then outputs of tile s - 2.
    const int steps = tiles + 1;
    for (int s = 0; tiles > 0 && s <= steps; ++s) {
      if (s < steps) {
        if (!mbar_wait(bar(kRawFull + s % kRawBuffers), (s / kRawBuffers) & 1U, abort_flag)) break;
        // raw rows 4 quad .. 4 quad + 5 (times t - 2 .. t + 3 of the thread's first row), 12 bytes each
        const unsigned char *const raw =
            smem + kRawOffset + (s % kRawBuffers) * kRawBytes + (4 * quad) * kRawStride + cp * 12;
        float x[6][6];
#pragma unroll
        for (int j = 0; j < 6; ++j) {
          const std::uint32_t *const words = reinterpret_cast<const std::uint32_t *>(raw + j * kRawStride);
#pragma unroll
          for (int w = 0; w < 3; ++w) {
            const std::uint32_t word = words[w];
            x[j][2 * w] = __uint_as_float(word << 16U);
            x[j][2 * w + 1] = __uint_as_float(word & 0xffff0000U);
          }
        }
        std::uint32_t u[4], g[4];  // per row: (channel 2cp, channel 2cp + 1)
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          float z[6];
#pragma unroll
          for (int column = 0; column < 6; ++column) {
            // fmaf with +0, not a multiply: the sign of a zero result must match the FMA chain
            float acc = fmaf(x[m][column], taps[column][0], 0.0F);
            acc = fmaf(x[m + 1][column], taps[column][1], acc);
            z[column] = fmaf(x[m + 2][column], taps[column][2], acc);
          }
          g[m] = round_pair_bf16(z[0], z[3]);
          const std::uint32_t x1 = round_pair_bf16(z[1], z[4]);
          const std::uint32_t v = round_pair_bf16(z[2], z[5]);
          u[m] = round_pair_bf16(__uint_as_float(x1 << 16U) * __uint_as_float(v << 16U),
                                 __uint_as_float(x1 & 0xffff0000U) * __uint_as_float(v & 0xffff0000U));
        }
        mbar_arrive(bar(kRawEmpty + s % kRawBuffers));  // the raw rows are in registers
        // decode history: the last taps - 1 values of u per channel, chronological (rows in front
        // of the range count too: a short window ends inside them)
        const int t_quad = t_first + (s - 1) * kTile + 4 * quad;
        if (p.inner_cache != nullptr && t_quad + 3 >= p.length - (p.taps - 1) && t_quad < p.length) {
#pragma unroll
          for (int m = 0; m < 4; ++m) {
            const int t_row = t_quad + m;
            if (t_row < 0 || t_row >= p.length || t_row < p.length - (p.taps - 1)) continue;
            const int slot = (p.taps - 1) - (p.length - t_row);
            p.inner_cache[static_cast<std::size_t>(c0 + 2 * cp) * (p.taps - 1) + slot] = __uint_as_float(u[m] << 16U);
            p.inner_cache[static_cast<std::size_t>(c0 + 2 * cp + 1) * (p.taps - 1) + slot] =
                __uint_as_float(u[m] & 0xffff0000U);
          }
        }
        // The images of step s replace those of step s - 3, which iteration s - 2 read and tiles
        // s - 4, s - 3 multiplied (this thread saw tile s - 3 finish in its iteration s - 1).
        if (s >= 2 && !mbar_wait(bar(kStepDone + (s & 1)), ((s - 2) >> 1) & 1U, abort_flag)) break;
        // [channel][time] images: u as the B operand (K block 2s + quad / 16 of the ring), the gate
        // beside it; four consecutive time steps of a channel are eight contiguous bytes
        const int k = (4 * quad) % 64;
        unsigned char *const block = smem + kRingOffset + ((2 * s + quad / 16) % kRingBlocks) * kBlockBytes;
        unsigned char *const gate_block = smem + kGateOffset + ((s % 3) * 2 + quad / 16) * kBlockBytes;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int channel = 2 * cp + e;
          const int offset = channel * 128 + (((k >> 3) ^ (channel & 7)) << 4) + (k & 7) * 2;
          const std::uint32_t selector = e == 0 ? 0x5410U : 0x7632U;
          *reinterpret_cast<uint2 *>(block + offset) =
              make_uint2(__byte_perm(u[0], u[1], selector), __byte_perm(u[2], u[3], selector));
          *reinterpret_cast<uint2 *>(gate_block + offset) =
              make_uint2(__byte_perm(g[0], g[1], selector), __byte_perm(g[2], g[3], selector));
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_arrive(bar(kBFull + (s & 1)));
        // stage step s + 2 into the buffer of step s - 1, once every worker has left that one
        if (s + 2 < steps) {
          if (s >= 1 && !mbar_wait(bar(kRawEmpty + (s - 1) % kRawBuffers), ((s - 1) / kRawBuffers) & 1U, abort_flag))
            break;
          stage_raw(s + 2);
        }
      }
      // ---- outputs of tile i = s - 2: its rows are those of step s - 1
      const int i = s - 2;
      if (i >= 0) {
        const int acc = i & 1;
        if (!mbar_wait(bar(kAccFull + acc), (i >> 1) & 1U, abort_flag)) break;
        // every worker's images of step s - 1 (the accumulator only proves the tensor core saw them)
        if (!mbar_wait(bar(kBFull + ((s - 1) & 1)), ((s - 1) >> 1) & 1U, abort_flag)) break;
        tc_fence_after();
        std::uint32_t sums[8];
        tmem_load_8(tmem_base + acc * kGroup + half * 8 + (static_cast<std::uint32_t>((warp & 3) * 32) << 16U), sums);
        tmem_load_wait();
        tc_fence_before();
        mbar_arrive(bar(kAccEmpty + acc));
        const int t = t_first + i * kTile + row;
        if (t < p.length) {
          const int k = row % 64;
          const unsigned char *const u_block =
              smem + kRingOffset + ((2 * (s - 1) + row / 64) % kRingBlocks) * kBlockBytes;
          const unsigned char *const g_block = smem + kGateOffset + (((s - 1) % 3) * 2 + row / 64) * kBlockBytes;
          float y[8];
          std::uint32_t u_bits[8];
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const int channel = half * 8 + c;
            const int offset = channel * 128 + (((k >> 3) ^ (channel & 7)) << 4) + (k & 7) * 2;
            u_bits[c] = *reinterpret_cast<const unsigned short *>(u_block + offset);
            const float gate = __uint_as_float(
                static_cast<std::uint32_t>(*reinterpret_cast<const unsigned short *>(g_block + offset)) << 16U);
            y[c] = rbf(fmaf(direct[c], __uint_as_float(u_bits[c] << 16U), __uint_as_float(sums[c]))) * gate;
          }
          *reinterpret_cast<uint4 *>(p.output + static_cast<std::size_t>(t) * p.width + c0 + half * 8) = make_uint4(
              round_pair_bf16(y[0], y[1]), round_pair_bf16(y[2], y[3]), round_pair_bf16(y[4], y[5]),
              round_pair_bf16(y[6], y[7]));
          if (p.pregate != nullptr)
            *reinterpret_cast<uint4 *>(p.pregate + static_cast<std::size_t>(t) * p.width + c0 + half * 8) =
                make_uint4(u_bits[0] | (u_bits[1] << 16U), u_bits[2] | (u_bits[3] << 16U),
                           u_bits[4] | (u_bits[5] << 16U), u_bits[6] | (u_bits[7] << 16U));
        }
      }
      mbar_arrive(bar(kStepDone + (s & 1)));  // this thread is done with iteration s
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0) {
    const unsigned long long start = global_timer_ns();
    while (global_timer_ns() - start < 200000ULL) __nanosleep(1000);
    if (threadIdx.x == 0) atomicOr(error_word, 1 | 4);  // bit 2: this kernel
  }
  if (warp == kMmaWarp) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(32U) : "memory");
  }
}

}  // namespace

bool gated_fir_tcgen05_applicable(const GatedFirArgs &a) {
  return a.projection != nullptr && a.short_filter != nullptr && a.short_taps == 3 && !a.cross_correlation &&
         !a.filter_is_f32 && a.taps > 32 && a.taps <= 128 && a.groups != 0 && a.width == a.groups * kGroup &&
         a.length > a.row_begin && a.length <= 0x7fff0000U &&
         (reinterpret_cast<std::uintptr_t>(a.projection) & 15U) == 0 &&
         (reinterpret_cast<std::uintptr_t>(a.output) & 15U) == 0 &&
         (a.pregate == nullptr || (reinterpret_cast<std::uintptr_t>(a.pregate) & 15U) == 0) &&
         (reinterpret_cast<std::uintptr_t>(a.short_filter) & 15U) == 0;
}

int gated_fir_tcgen05(const GatedFirArgs &a, cudaStream_t stream) {
  if (!gated_fir_tcgen05_applicable(a)) return fail(kInvalidArgument, "tensor-core FIR arguments are invalid");
  int status = kOk, sm_count = kSmCount;
  int *const error = tc::error_word(&status, &sm_count);
  if (error == nullptr) return status;
  static bool configured[64] = {};
  int device = 0;
  cudaGetDevice(&device);
  if (device >= 0 && device < 64 && !configured[device]) {
    if (cudaFuncSetAttribute(gated_fir_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) !=
        cudaSuccess)
      return fail(kCuda, "cannot raise the tensor-core FIR shared-memory limit");
    configured[device] = true;
  }
  TcParams p{};
  p.projection = static_cast<const bf16 *>(a.projection);
  p.short_filter = static_cast<const bf16 *>(a.short_filter);
  p.filter = static_cast<const bf16 *>(a.filter);
  p.direct = static_cast<const bf16 *>(a.direct);
  p.output = static_cast<bf16 *>(a.output);
  p.pregate = static_cast<bf16 *>(a.pregate);
  p.inner_cache = a.inner_cache;
  p.length = static_cast<int>(a.length);
  p.row_begin = static_cast<int>(a.row_begin);
  p.width = static_cast<int>(a.width);
  p.taps = static_cast<int>(a.taps);
  // Ranges per group: the split whose waves x (tiles per range + the tile rebuilt in front + about a
  // tile and a half of set-up: the Toeplitz strip, the pipeline fill) is least.
  const int all_tiles = static_cast<int>((a.length - a.row_begin + kTile - 1) / kTile);
  const long slots = 2L * sm_count;
  int best_parts = 1;
  long best_cost = -1;
  for (int parts = 1; parts <= 8 && parts <= all_tiles; ++parts) {
    const int per = (all_tiles + parts - 1) / parts;
    const long ctas = static_cast<long>((all_tiles + per - 1) / per) * static_cast<long>(a.groups);
    const long cost = ((ctas + slots - 1) / slots) * (2 * per + 5);
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      best_parts = parts;
    }
  }
  p.tiles_per_cta = (all_tiles + best_parts - 1) / best_parts;
  const dim3 grid(static_cast<unsigned int>((all_tiles + p.tiles_per_cta - 1) / p.tiles_per_cta),
                  static_cast<unsigned int>(a.groups));
  if (grid.y > 65535) return fail(kInvalidArgument, "tensor-core FIR has too many groups");
  gated_fir_tcgen05_kernel<<<grid, kThreadsTotal, kSmemBytes, stream>>>(p, error);
  return check_launch("tensor-core FIR kernel");
}

}  // namespace evob
