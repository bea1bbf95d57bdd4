// Causal prefill attention for head size 128 on the 5th-generation tensor
// cores, two CTAs per SM: softmax(Q K^T / sqrt(128)) V with query i seeing keys
// 0 .. prefix + i (the contract of upstream's FlashAttention-2 call,
// src/cuda/flash_attention.cu:199-441).
//
// The one-CTA-per-SM kernel (attention_tcgen05.cu) is a latency chain: its eight
// softmax warps walk TMEM load -> row maximum -> exchange -> exp2 -> P store in
// lock-step and the tensor core waits for them.  Here a CTA still owns 128 query
// rows of one head but
//   * walks 64-key tiles, so Q (32 KiB), two K stages and two V stages
//     (16 KiB each) are 96 KiB and two CTAs share an SM: while one CTA's
//     softmax runs, the other's MMAs do;
//   * keeps P in TMEM: the BF16 probabilities overwrite the first half of the
//     row's scores (tcgen05.st) and are the A operand of P_j V_j from there, so P
//     costs no shared-memory write, read or proxy fence - shared-memory bandwidth
//     (Q and K_j for the scores, V_j, the TMA writes) is what bounds the kernel;
//   * keeps O in TMEM for the whole walk: P_j V_j accumulates in place, and the
//     accumulator is rescaled (TMEM load, multiply, TMEM store) only when a
//     row's reference maximum moves up by more than 2^8 - rows whose reference
//     holds multiply by one.  A thread therefore carries no output accumulator
//     (the other kernel spends 64 registers and 64 FMAs per tile on it);
//   * the row's reference, not its running maximum, is what the probabilities
//     are taken against: p = 2^((s - ref) / sqrt(128) * log2 e) <= 2^8, the same
//     value after the final division by the row sum.
// Warp roles: warp 0 TMA producer (K and V two stages deep), warp 1 MMA issuer (one
// lane each), warps 2-5 softmax: a thread owns one query row - its TMEM lane -
// so the row maximum and the row sum are its own (no exchange between warps),
// with the scale-and-shift and the sums as packed F32 pairs.  Every wait is
// time-bounded and raises the sticky error word of the projection kernels.
#include <cuda.h>

#include "common.cuh"
#include "ops_internal.hpp"
#include "projection_featurizer.cuh"  // round_pair_bf16
#include "tcgen05.cuh"

namespace evob {
namespace {
using namespace tc;

constexpr int kRows = 128;                      // query rows per CTA = head dimensions
constexpr int kKeys = 64;                       // keys per tile
constexpr int kThreads = 64 + 128;              // TMA warp, MMA warp, four softmax warps (a thread = a query row)
constexpr int kQHalfBytes = kRows * 128;        // one 64-column box of Q: 128 rows x 128 bytes
constexpr int kQBytes = 2 * kQHalfBytes;
constexpr int kKvHalfBytes = kKeys * 128;       // one 64-column box of K or V: 64 keys x 128 bytes
constexpr int kKvBytes = 2 * kKvHalfBytes;
constexpr int kQOffset = 0;
constexpr int kKOffset = kQOffset + kQBytes;    // two stages
constexpr int kVOffset = kKOffset + 2 * kKvBytes;  // two stages
constexpr int kBarrierOffset = kVOffset + 2 * kKvBytes;
enum Barrier : int {
  kQFull = 0, kKFull = 1, kKEmpty = 3, kVFull = 5, kVEmpty = 7, kSFull = 9, kPFull = 11, kOFull = 12, kBarriers = 13
};
constexpr int kTmemPtrOffset = kBarrierOffset + kBarriers * 8;
constexpr int kAbortOffset = kTmemPtrOffset + 8;
constexpr int kSmemBytes = kAbortOffset + 16;  // no slack: the kernel checks the 1024-byte alignment it asked for
static_assert(2 * (kSmemBytes + 1024) <= 228 * 1024, "two CTAs per SM");
constexpr std::uint32_t kTmemColumns = 256;  // S0 | S1 (64 each; P_j replaces the first 32 columns of S_j) | O (128)
constexpr std::uint32_t kScoreColumns = kKeys;
// A reference maximum is replaced only when the tile's maximum exceeds it by this many doublings.
constexpr float kLazyDoublings = 8.0F;

// V tile as the B operand of O += P V: N (head dimension) is the contiguous
// direction.  64-column boxes are one box apart (leading offset), groups of
// eight keys 1 KiB apart (stride offset).
__device__ __forceinline__ std::uint64_t v_descriptor(const std::uint32_t address) {
  std::uint64_t desc = 0;
  desc |= static_cast<std::uint64_t>((address & 0x3ffffU) >> 4U);
  desc |= static_cast<std::uint64_t>(kKvHalfBytes >> 4U) << 16U;  // LBO
  desc |= static_cast<std::uint64_t>(1024U >> 4U) << 32U;         // SBO
  desc |= static_cast<std::uint64_t>(1U) << 46U;                  // version
  desc |= static_cast<std::uint64_t>(2U) << 61U;                  // SWIZZLE_128B
  return desc;
}

__host__ __device__ constexpr std::uint32_t instruction_descriptor(const int n, const bool b_mn_major) {
  std::uint32_t d = 0;
  d |= 1U << 4U;                       // accumulator F32
  d |= 1U << 7U;                       // A BF16
  d |= 1U << 10U;                      // B BF16
  d |= (b_mn_major ? 1U : 0U) << 16U;  // B major
  d |= static_cast<std::uint32_t>(n >> 3) << 17U;
  d |= static_cast<std::uint32_t>(kRows >> 4) << 24U;  // M = 128
  return d;
}

__device__ __forceinline__ float max3(const float a, const float b, const float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float fast_exp2(const float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// D[tmem] (+)= A[tmem] * B[smem]: the A operand (M x 16 BF16, two per 32-bit column) is read from
// tensor memory.
__device__ __forceinline__ void tc_mma_a_tmem(const std::uint32_t tmem_d, const std::uint32_t tmem_a,
                                              const std::uint64_t desc_b, const std::uint32_t idesc,
                                              const std::uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_store_32(const std::uint32_t taddr, const std::uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
      "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]),
      "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]),
      "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
// Packed F32 pairs: one instruction for two lanes of F32 arithmetic.
__device__ __forceinline__ unsigned long long pack_f32x2(const float low, const float high) {
  unsigned long long d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(low), "f"(high));
  return d;
}
__device__ __forceinline__ void unpack_f32x2(const unsigned long long pair, float &low, float &high) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(low), "=f"(high) : "l"(pair));
}
__device__ __forceinline__ unsigned long long fma_f32x2(const unsigned long long a, const unsigned long long b,
                                                        const unsigned long long c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ unsigned long long add_f32x2(const unsigned long long a, const unsigned long long b) {
  unsigned long long d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ void tmem_load_16(const std::uint32_t taddr, std::uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_store_16(const std::uint32_t taddr, const std::uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
      "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
__device__ __forceinline__ void tmem_store_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__global__ void __launch_bounds__(kThreads, 2)
flash_tcgen05_k64_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, bf16 *const output, const int rows,
                         const int total_keys, const int heads, int *const error_word) {
  extern __shared__ __align__(1024) unsigned char smem[];
  const std::uint32_t smem_base = smem_u32(smem);
  auto bar = [&](const int index) { return smem_base + kBarrierOffset + 8U * index; };
  volatile std::uint32_t *const tmem_ptr = reinterpret_cast<volatile std::uint32_t *>(smem + kTmemPtrOffset);
  volatile int *const abort_flag = reinterpret_cast<volatile int *>(smem + kAbortOffset);
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;

  // heaviest query blocks first
  const int q_block = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
  const int head = blockIdx.y;
  const int q0 = q_block * kRows;
  const int prefix = total_keys - rows;
  // keys this block may see: 0 .. prefix + q0 + 127, inside the cache
  const int visible = min(total_keys, prefix + q0 + kRows);
  const int tiles = (visible + kKeys - 1) / kKeys;

  if (threadIdx.x == 0) {
    mbar_init(bar(kQFull), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(kKFull + s), 1);
      mbar_init(bar(kKEmpty + s), 1);
      mbar_init(bar(kVFull + s), 1);
      mbar_init(bar(kVEmpty + s), 1);
      mbar_init(bar(kSFull + s), 1);
    }
    mbar_init(bar(kPFull), 4);
    mbar_init(bar(kOFull), 1);
    *abort_flag = (smem_base & 1023U) != 0U ? 1 : 0;  // the tiles need the alignment the declaration asks for
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(const_cast<std::uint32_t *>(tmem_ptr))),
                 "r"(kTmemColumns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const std::uint32_t tmem_base = *tmem_ptr;
  const std::uint32_t tmem_o = tmem_base + 2 * kScoreColumns;
  const bool aligned = *abort_flag == 0;

  if (!aligned) {
    // nothing is issued; the error word is raised below
  } else if (warp == 0) {
    if (lane == 0) {
      const int column = head * kRows;
      mbar_expect_tx(bar(kQFull), kQBytes);
      tma_load_2d(smem_base + kQOffset, &map_q, bar(kQFull), column, q0);
      tma_load_2d(smem_base + kQOffset + kQHalfBytes, &map_q, bar(kQFull), column + 64, q0);
      for (int j = 0; j < tiles; ++j) {
        const int s = j & 1;
        const std::uint32_t phase = (j >> 1) & 1U;
        if (!mbar_wait(bar(kKEmpty + s), phase ^ 1U, abort_flag)) break;
        const std::uint32_t k_dst = smem_base + kKOffset + s * kKvBytes;
        mbar_expect_tx(bar(kKFull + s), kKvBytes);
        tma_load_2d(k_dst, &map_k, bar(kKFull + s), column, j * kKeys);
        tma_load_2d(k_dst + kKvHalfBytes, &map_k, bar(kKFull + s), column + 64, j * kKeys);
        if (!mbar_wait(bar(kVEmpty + s), phase ^ 1U, abort_flag)) break;
        const std::uint32_t v_dst = smem_base + kVOffset + s * kKvBytes;
        mbar_expect_tx(bar(kVFull + s), kKvBytes);
        tma_load_2d(v_dst, &map_v, bar(kVFull + s), column, j * kKeys);
        tma_load_2d(v_dst + kKvHalfBytes, &map_v, bar(kVFull + s), column + 64, j * kKeys);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr std::uint32_t idesc_scores = instruction_descriptor(kKeys, false);
      constexpr std::uint32_t idesc_output = instruction_descriptor(kRows, true);
      bool ok = mbar_wait(bar(kQFull), 0U, abort_flag);
      // S_j = Q K_j^T (M128 N64, K = 128 dimensions in eight k16 steps) into score buffer j & 1.
      // P_{j-2} sat in that buffer: its P V must have finished (which also means the scores of
      // tile j - 2 were read long ago).
      auto issue_scores = [&](const int j) -> bool {
        const int s = j & 1;
        if (!mbar_wait(bar(kKFull + s), (j >> 1) & 1U, abort_flag)) return false;
        if (j >= 2 && !mbar_wait(bar(kOFull), (j - 2) & 1U, abort_flag)) return false;
        tc_fence_after();
        const std::uint32_t k_base = smem_base + kKOffset + s * kKvBytes;
#pragma unroll
        for (int k = 0; k < 8; ++k)
          tc_mma<false>(tmem_base + s * kScoreColumns,
                        smem_descriptor(smem_base + kQOffset + (k / 4) * kQHalfBytes + (k % 4) * 32),
                        smem_descriptor(k_base + (k / 4) * kKvHalfBytes + (k % 4) * 32), idesc_scores,
                        k != 0 ? 1U : 0U);
        tc_commit(bar(kKEmpty + s));
        tc_commit(bar(kSFull + s));
        return true;
      };
      if (ok) ok = issue_scores(0);
      for (int j = 0; j < tiles && ok; ++j) {
        if (j + 1 < tiles && !issue_scores(j + 1)) break;
        const int s = j & 1;
        if (!mbar_wait(bar(kVFull + s), (j >> 1) & 1U, abort_flag)) break;
        // P_j is in tensor memory, and O is rescaled where a row needed it
        if (!mbar_wait(bar(kPFull), j & 1U, abort_flag)) break;
        tc_fence_after();
        const std::uint32_t v_base = smem_base + kVOffset + s * kKvBytes;
#pragma unroll
        for (int k = 0; k < kKeys / 16; ++k)
          // A: 16 keys of P (eight 32-bit columns of tensor memory); B: 16 key rows of V
          tc_mma_a_tmem(tmem_o, tmem_base + s * kScoreColumns + k * 8, v_descriptor(v_base + k * 16 * 128),
                        idesc_output, (j | k) != 0 ? 1U : 0U);
        tc_commit(bar(kVEmpty + s));
        tc_commit(bar(kOFull));
      }
    }
  } else {
    const int quarter = warp % 4;
    const int row = quarter * 32 + lane;  // query row inside the block = TMEM lane
    const std::uint32_t lane_base = static_cast<std::uint32_t>(quarter * 32) << 16U;
    const int position = prefix + q0 + row;  // last key this row may see
    const float scale_log2 = 1.4426950408889634F * rsqrtf(static_cast<float>(kRows));
    const float slack = kLazyDoublings / scale_log2;  // in score units
    const unsigned long long scale_pair = pack_f32x2(scale_log2, scale_log2);
    float reference = -INFINITY, running_sum = 0.0F;
    bool ok = true;

    for (int j = 0; j < tiles; ++j) {
      const int s = j & 1;
      if (!mbar_wait(bar(kSFull + s), (j >> 1) & 1U, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after();
      std::uint32_t v[kKeys];
      {
        std::uint32_t chunk[2][32];
        tmem_load_32(tmem_base + s * kScoreColumns + lane_base, chunk[0]);
        tmem_load_32(tmem_base + s * kScoreColumns + lane_base + 32, chunk[1]);
        tmem_load_wait();
#pragma unroll
        for (int i = 0; i < kKeys; ++i) v[i] = chunk[i / 32][i % 32];
      }
      if (j * kKeys + kKeys - 1 > prefix + q0) {     // some key hidden from some row
#pragma unroll
        for (int i = 0; i < kKeys; ++i)
          if (j * kKeys + i > position) v[i] = 0xff800000U;  // -inf
      }
      float partial_max[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < kKeys; i += 2)
        partial_max[(i / 2) % 4] = max3(partial_max[(i / 2) % 4], __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
      const float tile_max = fmaxf(fmaxf(partial_max[0], partial_max[1]), fmaxf(partial_max[2], partial_max[3]));
      const bool moved = tile_max > reference + slack;  // true on the first tile: reference = -inf
      const float alpha = moved ? fast_exp2((reference - tile_max) * scale_log2) : 1.0F;
      if (moved) reference = tile_max;
      const float bias = -reference * scale_log2;
      const unsigned long long bias_pair = pack_f32x2(bias, bias);
      // probabilities and the row sum first: they need nothing from the previous tile's P V
      unsigned long long partial_sum[4] = {0ULL, 0ULL, 0ULL, 0ULL};  // (even key, odd key) pairs of F32 sums
      std::uint32_t packed[kKeys / 2];
      // in three sweeps, so that no instruction waits for the one before it
      float t[kKeys];
#pragma unroll
      for (int i = 0; i < kKeys; i += 2)
        unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(v[i]), __uint_as_float(v[i + 1])), scale_pair, bias_pair),
                     t[i], t[i + 1]);
#pragma unroll
      for (int i = 0; i < kKeys; ++i) t[i] = fast_exp2(t[i]);
#pragma unroll
      for (int i = 0; i < kKeys; i += 2) {
        partial_sum[(i / 2) % 4] = add_f32x2(partial_sum[(i / 2) % 4], pack_f32x2(t[i], t[i + 1]));
        packed[i / 2] = round_pair_bf16(t[i], t[i + 1]);
      }
      partial_sum[0] = add_f32x2(partial_sum[0], partial_sum[2]);
      partial_sum[1] = add_f32x2(partial_sum[1], partial_sum[3]);
      float sum_even, sum_odd, sum_even_b, sum_odd_b;
      unpack_f32x2(partial_sum[0], sum_even, sum_odd);
      unpack_f32x2(partial_sum[1], sum_even_b, sum_odd_b);
      running_sum = fmaf(running_sum, alpha, (sum_even + sum_odd) + (sum_even_b + sum_odd_b));
      if (j > 0) {
        // Every warp follows the O-ready barrier tile by tile, whether it has to rescale or not: a parity
        // wait cannot tell a phase from the one two before or two after it, so a waiter that skipped
        // phases would either run ahead of a P V that has not finished or wait for one that finished
        // long ago.  Having seen P V of tile j - 1 finish also means every warp has stored its
        // probabilities of tile j - 1 (an mbarrier does not know which tile an arrival belongs to: no
        // warp may arrive for tile j while the phase of tile j - 1 is still open).
        if (!mbar_wait(bar(kOFull), (j - 1) & 1U, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (__any_sync(0xffffffffU, moved)) {
#pragma unroll
          for (int c = 0; c < kRows / 16; ++c) {
            std::uint32_t o[16];
            const std::uint32_t address = tmem_o + lane_base + c * 16;
            tmem_load_16(address, o);
            tmem_load_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_store_16(address, o);
          }
        }
      }
      // BF16 P over the first 32 columns of this row's scores (all 64 are in registers by now)
      tmem_store_32(tmem_base + s * kScoreColumns + lane_base, packed);
      tmem_store_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kPFull));
    }
    if (ok && tiles > 0 && mbar_wait(bar(kOFull), (tiles - 1) & 1U, abort_flag)) {
      tc_fence_after();
      const float inverse = 1.0F / running_sum;
      bf16 *const out = output + static_cast<std::size_t>(q0 + row) * (static_cast<std::size_t>(heads) * kRows) +
                        static_cast<std::size_t>(head) * kRows;
#pragma unroll
      for (int c = 0; c < kRows / 32; ++c) {
        std::uint32_t o[32];
        tmem_load_32(tmem_o + lane_base + c * 32, o);  // warp-wide: before the row test
        tmem_load_wait();
        if (q0 + row < rows) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 word;
            word.x = round_pair_bf16(__uint_as_float(o[8 * q]) * inverse, __uint_as_float(o[8 * q + 1]) * inverse);
            word.y = round_pair_bf16(__uint_as_float(o[8 * q + 2]) * inverse, __uint_as_float(o[8 * q + 3]) * inverse);
            word.z = round_pair_bf16(__uint_as_float(o[8 * q + 4]) * inverse, __uint_as_float(o[8 * q + 5]) * inverse);
            word.w = round_pair_bf16(__uint_as_float(o[8 * q + 6]) * inverse, __uint_as_float(o[8 * q + 7]) * inverse);
            *reinterpret_cast<uint4 *>(out + c * 32 + 8 * q) = word;
          }
        }
      }
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0) {
    // let copies that may still be in flight land before the shared memory is recycled
    // (also reached when the dynamic shared memory did not start on a 1024-byte boundary)
    const unsigned long long start = global_timer_ns();
    while (global_timer_ns() - start < 200000ULL) __nanosleep(1000);
    if (threadIdx.x == 0) atomicOr(error_word, 1 | 8);  // bit 3: this kernel
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColumns)
                 : "memory");
  }
}

}  // namespace

int flash_tcgen05_attention_k64(const void *query, const void *key_cache, const void *value_cache,
                                const std::size_t rows, const std::size_t total_keys, const std::size_t heads,
                                void *output, cudaStream_t stream) {
  int status = kOk;
  int *const error = tc::error_word(&status, nullptr);
  if (error == nullptr) return status;
  const std::size_t width = heads * kRows;
  CUtensorMap map_q, map_k, map_v;
  if ((status = tc::make_bf16_tile_map(&map_q, query, rows, width, kRows)) != kOk ||
      (status = tc::make_bf16_tile_map(&map_k, key_cache, total_keys, width, kKeys)) != kOk ||
      (status = tc::make_bf16_tile_map(&map_v, value_cache, total_keys, width, kKeys)) != kOk)
    return status;
  if (cudaFuncSetAttribute(flash_tcgen05_k64_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) !=
          cudaSuccess ||
      cudaFuncSetAttribute(flash_tcgen05_k64_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                           cudaSharedmemCarveoutMaxShared) != cudaSuccess)
    return fail(kCuda, "cannot raise the attention shared-memory limit");
  const dim3 grid(ceil_div_u(rows, kRows), static_cast<unsigned int>(heads));
  flash_tcgen05_k64_kernel<<<grid, kThreads, kSmemBytes, stream>>>(map_q, map_k, map_v, static_cast<bf16 *>(output),
                                                                  static_cast<int>(rows), static_cast<int>(total_keys),
                                                                  static_cast<int>(heads), error);
  return check_launch("tcgen05 attention kernel (64-key tiles)");
}

}  // namespace evob
