// Causal prefill attention for head size 128 on the 5th-generation tensor
// cores: softmax(Q K^T / sqrt(128)) V with query i seeing keys 0 .. prefix + i
// (the contract of upstream's FlashAttention-2 call,
// src/cuda/flash_attention.cu:199-441).
//
// One CTA owns 128 query rows of one head and walks the 128-key K/V tiles it
// may see.  Warp roles:
//   warp 0     TMA producer: Q once, then K_j and V_j tiles (two 64-column
//              boxes each, 128-byte swizzle) into 2-deep rings.
//   warp 1     MMA issuer (one lane): S_j = Q K_j^T (M128 N128, K = 128 dims in
//              eight k16 steps) into one of two TMEM score buffers, issued one
//              tile ahead of the softmax; then O_j = P_j V_j with P_j read
//              from shared memory (K-major) and V_j used in place as an
//              MN-major operand, into a third TMEM buffer.
//   warps 2-17 softmax: a thread owns a quarter of one query row (its TMEM
//              lane; four warps share a lane quarter and split the 128 columns), so
//              row maxima and sums need no shuffles - the four parts exchange
//              one maximum per tile through shared memory.  Scores are read
//              from TMEM once and kept in registers (max, then exp2 / sum /
//              BF16 pack), P_j written to shared memory in the swizzled K-major layout, O_j
//              added into a register accumulator with the usual running-max
//              rescale.
// Score buffers, the P tile and the O_j buffer are handed back and forth with
// mbarriers; every wait is time-bounded and raises the same sticky error word
// as the projection kernels.
#include <cuda.h>

#include <cstdlib>

#include "common.cuh"
#include "ops_internal.hpp"
#include "projection_featurizer.cuh"
#include "tcgen05.cuh"

namespace evob {
namespace {
using namespace tc;

constexpr int kSides = 2;                         // softmax warps per TMEM lane quarter
constexpr int kSideColumns = 128 / kSides;        // keys / output dimensions per softmax warp and tile
constexpr int kThreads = 64 + 128 * kSides;       // TMA warp, MMA warp, 4 * kSides softmax warps
constexpr int kSideChunks = kSideColumns / 32;    // 32-column TMEM loads per softmax thread and tile
static_assert(kSideColumns % 32 == 0 && kSideColumns <= 64, "sides are one or two 32-column TMEM loads");
constexpr int kTile = 128;                    // query rows per CTA and keys per tile
constexpr int kHalfBytes = kTile * 128;       // one 64-column box: 128 rows x 128 bytes
constexpr int kTileBytes = 2 * kHalfBytes;    // 32 KiB
constexpr int kQOffset = 0;
constexpr int kKOffset = kTileBytes;                    // 2 stages
constexpr int kVOffset = kKOffset + 2 * kTileBytes;     // 2 stages
constexpr int kPOffset = kVOffset + 2 * kTileBytes;
constexpr int kBarrierOffset = kPOffset + kTileBytes;
constexpr int kBarriers = 21;
constexpr int kTmemPtrOffset = kBarrierOffset + kBarriers * 8;
constexpr int kAbortOffset = kTmemPtrOffset + 8;
constexpr int kExchangeOffset = kAbortOffset + 16;                // 2 x 2 x 128 floats
constexpr int kSmemBytes = kExchangeOffset + 2 * kSides * kTile * 4 + 1024;  // + alignment slack
constexpr std::uint32_t kTmemColumns = 512;            // S0 | S1 | O | unused
constexpr std::uint32_t kScoreColumns = 128;

enum Barrier : int {
  kQFull = 0, kKFull = 1, kKEmpty = 3, kVFull = 5, kVEmpty = 7, kSFull = 9, kSEmpty = 11,
  kPFull = 13, kOFull = 14, kOEmpty = 15, kMaxReady = 16 /* one per lane quarter */, kSumReady = 20
};

// V tile as the B operand of O = P V: N (head dimension) is the contiguous
// direction.  64-column boxes are 16 KiB apart (leading offset), groups of
// eight keys 1 KiB apart (stride offset).
__device__ __forceinline__ std::uint64_t mn_major_descriptor(const std::uint32_t address) {
  std::uint64_t desc = 0;
  desc |= static_cast<std::uint64_t>((address & 0x3ffffU) >> 4U);
  desc |= static_cast<std::uint64_t>(kHalfBytes >> 4U) << 16U;  // LBO
  desc |= static_cast<std::uint64_t>(1024U >> 4U) << 32U;       // SBO
  desc |= static_cast<std::uint64_t>(1U) << 46U;                // version
  desc |= static_cast<std::uint64_t>(2U) << 61U;                // SWIZZLE_128B
  return desc;
}

__host__ __device__ constexpr std::uint32_t instruction_descriptor(const bool b_mn_major) {
  std::uint32_t d = 0;
  d |= 1U << 4U;                            // accumulator F32
  d |= 1U << 7U;                            // A BF16
  d |= 1U << 10U;                           // B BF16
  d |= (b_mn_major ? 1U : 0U) << 16U;       // B major
  d |= static_cast<std::uint32_t>(kTile >> 3) << 17U;  // N = 128
  d |= static_cast<std::uint32_t>(kTile >> 4) << 24U;  // M = 128
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

__global__ void __launch_bounds__(kThreads, 1)
flash_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_v, bf16 *const output, const int rows,
                     const int total_keys, const int heads, int *const error_word) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char *const smem = smem_raw + ((1024U - (smem_u32(smem_raw) & 1023U)) & 1023U)  /* pointer arithmetic keeps the shared address space */;
  const std::uint32_t smem_base = smem_u32(smem);
  auto bar = [&](const int index) { return smem_base + kBarrierOffset + 8U * index; };
  volatile std::uint32_t *const tmem_ptr = reinterpret_cast<volatile std::uint32_t *>(smem + kTmemPtrOffset);
  volatile int *const abort_flag = reinterpret_cast<volatile int *>(smem + kAbortOffset);
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;

  // heaviest query blocks first
  const int q_block = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
  const int head = blockIdx.y;
  const int q0 = q_block * kTile;
  const int prefix = total_keys - rows;
  // keys this block may see: 0 .. prefix + q0 + 127, inside the cache
  const int visible = min(total_keys, prefix + q0 + kTile);
  const int tiles = (visible + kTile - 1) / kTile;

  if (threadIdx.x == 0) {
    mbar_init(bar(kQFull), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(kKFull + s), 1);
      mbar_init(bar(kKEmpty + s), 1);
      mbar_init(bar(kVFull + s), 1);
      mbar_init(bar(kVEmpty + s), 1);
      mbar_init(bar(kSFull + s), 1);
      mbar_init(bar(kSEmpty + s), 4 * kSides);
    }
    mbar_init(bar(kPFull), 4 * kSides);
    mbar_init(bar(kOFull), 1);
    mbar_init(bar(kOEmpty), 4 * kSides);
    for (int q = 0; q < 4; ++q) mbar_init(bar(kMaxReady + q), kSides);
    mbar_init(bar(kSumReady), 4 * kSides);
    *abort_flag = 0;
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

  if (warp == 0) {
    if (lane == 0) {
      const int column = head * kTile;
      mbar_expect_tx(bar(kQFull), kTileBytes);
      tma_load_2d(smem_base + kQOffset, &map_q, bar(kQFull), column, q0);
      tma_load_2d(smem_base + kQOffset + kHalfBytes, &map_q, bar(kQFull), column + 64, q0);
      for (int j = 0; j < tiles; ++j) {
        const int s = j & 1;
        const std::uint32_t phase = (j >> 1) & 1U;
        if (!mbar_wait(bar(kKEmpty + s), phase ^ 1U, abort_flag)) break;
        const std::uint32_t k_dst = smem_base + kKOffset + s * kTileBytes;
        mbar_expect_tx(bar(kKFull + s), kTileBytes);
        tma_load_2d(k_dst, &map_k, bar(kKFull + s), column, j * kTile);
        tma_load_2d(k_dst + kHalfBytes, &map_k, bar(kKFull + s), column + 64, j * kTile);
        if (!mbar_wait(bar(kVEmpty + s), phase ^ 1U, abort_flag)) break;
        const std::uint32_t v_dst = smem_base + kVOffset + s * kTileBytes;
        mbar_expect_tx(bar(kVFull + s), kTileBytes);
        tma_load_2d(v_dst, &map_v, bar(kVFull + s), column, j * kTile);
        tma_load_2d(v_dst + kHalfBytes, &map_v, bar(kVFull + s), column + 64, j * kTile);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr std::uint32_t idesc_scores = instruction_descriptor(false);
      constexpr std::uint32_t idesc_output = instruction_descriptor(true);
      bool ok = mbar_wait(bar(kQFull), 0U, abort_flag);
      // S_j = Q K_j^T into score buffer j & 1
      auto issue_scores = [&](const int j) -> bool {
        const int s = j & 1;
        const std::uint32_t phase = (j >> 1) & 1U;
        if (!mbar_wait(bar(kKFull + s), phase, abort_flag)) return false;
        if (!mbar_wait(bar(kSEmpty + s), phase ^ 1U, abort_flag)) return false;
        tc_fence_after();
        const std::uint32_t k_base = smem_base + kKOffset + s * kTileBytes;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const std::uint32_t offset = (k / 4) * kHalfBytes + (k % 4) * 32;
          tc_mma<false>(tmem_base + s * kScoreColumns, smem_descriptor(smem_base + kQOffset + offset),
                        smem_descriptor(k_base + offset), idesc_scores, k != 0 ? 1U : 0U);
        }
        tc_commit(bar(kKEmpty + s));
        tc_commit(bar(kSFull + s));
        return true;
      };
      if (ok) ok = issue_scores(0);
      for (int j = 0; j < tiles && ok; ++j) {
        if (j + 1 < tiles && !issue_scores(j + 1)) break;
        const int s = j & 1;
        if (!mbar_wait(bar(kVFull + s), (j >> 1) & 1U, abort_flag)) break;
        if (!mbar_wait(bar(kPFull), j & 1U, abort_flag)) break;
        if (!mbar_wait(bar(kOEmpty), (j & 1U) ^ 1U, abort_flag)) break;
        tc_fence_after();
        const std::uint32_t v_base = smem_base + kVOffset + s * kTileBytes;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          // A: 16 keys of P (K-major, 32 bytes inside the swizzle row); B: 16 key rows of V
          const std::uint32_t p_offset = (k / 4) * kHalfBytes + (k % 4) * 32;
          tc_mma<false>(tmem_o, smem_descriptor(smem_base + kPOffset + p_offset),
                        mn_major_descriptor(v_base + k * 16 * 128), idesc_output, k != 0 ? 1U : 0U);
        }
        tc_commit(bar(kVEmpty + s));
        tc_commit(bar(kOFull));
      }
    }
  } else {
    // kSides softmax warps share each TMEM lane quarter and split the columns:
    // side s takes keys / output dimensions s*kSideColumns .. of every tile.  A
    // row's maximum is the one value the sides exchange per tile (through
    // shared memory, behind a bounded mbarrier wait).
    const int quarter = warp % 4;
    const int side = (warp - 2) / 4;
    const int row = quarter * 32 + lane;                    // query row inside the block = TMEM lane
    const std::uint32_t lane_base = static_cast<std::uint32_t>(quarter * 32) << 16U;
    const std::uint32_t column_base = static_cast<std::uint32_t>(side * kSideColumns);
    const int position = prefix + q0 + row;                 // last key this row may see
    const float scale_log2 = 1.4426950408889634F * rsqrtf(static_cast<float>(kTile));
    float accumulator[kSideColumns];
#pragma unroll
    for (int i = 0; i < kSideColumns; ++i) accumulator[i] = 0.0F;
    float running_max = -INFINITY, running_sum = 0.0F, previous_alpha = 1.0F;
    // this side's keys of the row: 16-byte chunks first_chunk .. of one 64-key half of the P tile
    unsigned char *const p_row = smem + kPOffset + (side * kSideColumns / 64) * kHalfBytes + row * 128;
    const int first_chunk = (side * kSideColumns % 64) / 8;
    float *const exchange = reinterpret_cast<float *>(smem + kExchangeOffset);  // [2 tiles][kSides][128 rows]
    bool ok = true;

    // O_reg = O_reg * alpha + (P V of the tile that just finished)
    auto absorb_output = [&](const float alpha) {
      std::uint32_t v[kSideChunks][32];
#pragma unroll
      for (int c = 0; c < kSideChunks; ++c) tmem_load_32(tmem_o + lane_base + column_base + c * 32, v[c]);
      tmem_load_wait();
#pragma unroll
      for (int c = 0; c < kSideChunks; ++c)
#pragma unroll
        for (int i = 0; i < 32; ++i)
          accumulator[c * 32 + i] = fmaf(accumulator[c * 32 + i], alpha, __uint_as_float(v[c][i]));
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kOEmpty));
    };

    for (int j = 0; j < tiles; ++j) {
      const int s = j & 1;
      if (!mbar_wait(bar(kSFull + s), (j >> 1) & 1U, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int key0 = j * kTile + side * kSideColumns;
      const bool boundary = j * kTile + kTile - 1 > prefix + q0;  // some key hidden from some row
      // this side's scores stay in registers from here to the P store
      std::uint32_t v[kSideColumns];
      {
        std::uint32_t chunk[kSideChunks][32];
#pragma unroll
        for (int c = 0; c < kSideChunks; ++c)
          tmem_load_32(tmem_base + s * kScoreColumns + lane_base + column_base + c * 32, chunk[c]);
        tmem_load_wait();
#pragma unroll
        for (int c = 0; c < kSideChunks; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) v[c * 32 + i] = chunk[c][i];
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kSEmpty + s));  // the score buffer may be overwritten
      if (boundary) {
#pragma unroll
        for (int i = 0; i < kSideColumns; ++i)
          if (key0 + i > position) v[i] = 0xff800000U;  // -inf
      }
      float partial_max[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < kSideColumns; i += 2)
        partial_max[(i / 2) % 4] = max3(partial_max[(i / 2) % 4], __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
      const float side_max = fmaxf(fmaxf(partial_max[0], partial_max[1]), fmaxf(partial_max[2], partial_max[3]));
      exchange[(s * kSides + side) * kTile + row] = side_max;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kMaxReady + quarter));
      if (!mbar_wait(bar(kMaxReady + quarter), j & 1U, abort_flag)) {
        ok = false;
        break;
      }
      float tile_max = side_max;
#pragma unroll
      for (int other = 1; other < kSides; ++other)
        tile_max = fmaxf(tile_max, exchange[(s * kSides + ((side + other) % kSides)) * kTile + row]);
      const float new_max = fmaxf(running_max, tile_max);
      const float alpha = fast_exp2((running_max - new_max) * scale_log2);
      const float bias = -new_max * scale_log2;
      if (j > 0) {
        // P V of the previous tile: frees the P tile and delivers O_{j-1}
        if (!mbar_wait(bar(kOFull), (j - 1) & 1U, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        absorb_output(previous_alpha);
      }
      // probabilities, partial row sum, BF16 pack into the swizzled P tile
      float partial_sum[4] = {0.0F, 0.0F, 0.0F, 0.0F};
      std::uint32_t packed[kSideColumns / 2];
#pragma unroll
      for (int i = 0; i < kSideColumns; i += 2) {
        const float px = fast_exp2(fmaf(__uint_as_float(v[i]), scale_log2, bias));
        const float py = fast_exp2(fmaf(__uint_as_float(v[i + 1]), scale_log2, bias));
        partial_sum[(i / 2) % 4] += px + py;
        // BF16 by integer round-half-up (probabilities are finite and >= 0): keeps
        // the conversion off the transcendental unit, which the exp2 above saturates
        packed[i / 2] = __byte_perm(__float_as_uint(px) + 0x8000U, __float_as_uint(py) + 0x8000U, 0x7632);
      }
#pragma unroll
      for (int q = 0; q < kSideColumns / 8; ++q)
        *reinterpret_cast<uint4 *>(p_row + (((first_chunk + q) ^ (row & 7)) << 4)) =
            make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
      // P visible to the tensor core (async proxy)
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kPFull));
      running_sum = fmaf(running_sum, alpha, (partial_sum[0] + partial_sum[1]) + (partial_sum[2] + partial_sum[3]));
      running_max = new_max;
      previous_alpha = alpha;
    }
    if (ok && tiles > 0 && mbar_wait(bar(kOFull), (tiles - 1) & 1U, abort_flag)) {
      tc_fence_after();
      absorb_output(previous_alpha);
      // the row sum is the sum of the sides' partial sums
      exchange[side * kTile + row] = running_sum;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kSumReady));
      if (mbar_wait(bar(kSumReady), 0U, abort_flag) && q0 + row < rows) {
        float total = 0.0F;
#pragma unroll
        for (int other = 0; other < kSides; ++other) total += exchange[other * kTile + row];
        const float inverse = 1.0F / total;
        bf16 *const out = output + static_cast<std::size_t>(q0 + row) * (static_cast<std::size_t>(heads) * kTile) +
                          static_cast<std::size_t>(head) * kTile + side * kSideColumns;
#pragma unroll
        for (int q = 0; q < kSideColumns / 8; ++q) {
          uint4 word;
          word.x = round_pair_bf16(accumulator[8 * q] * inverse, accumulator[8 * q + 1] * inverse);
          word.y = round_pair_bf16(accumulator[8 * q + 2] * inverse, accumulator[8 * q + 3] * inverse);
          word.z = round_pair_bf16(accumulator[8 * q + 4] * inverse, accumulator[8 * q + 5] * inverse);
          word.w = round_pair_bf16(accumulator[8 * q + 6] * inverse, accumulator[8 * q + 7] * inverse);
          *reinterpret_cast<uint4 *>(out + 8 * q) = word;
        }
      }
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0) {
    // let copies that may still be in flight land before the shared memory is recycled
    const unsigned long long start = global_timer_ns();
    while (global_timer_ns() - start < 200000ULL) __nanosleep(1000);
    if (threadIdx.x == 0) atomicOr(error_word, 1 | 16);  // bit 4: this kernel
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColumns)
                 : "memory");
  }
}

}  // namespace

// attention_tcgen05_k64.cu: the same contract on 64-key tiles, two CTAs per SM, O kept in TMEM
int flash_tcgen05_attention_k64(const void *query, const void *key_cache, const void *value_cache, std::size_t rows,
                                std::size_t total_keys, std::size_t heads, void *output, cudaStream_t stream);

bool flash_tcgen05_applicable(const void *query, const void *key_cache, const void *value_cache,
                              const std::size_t rows, const std::size_t total_keys, const std::size_t heads,
                              const void *output) {
  if (rows < kTile || heads == 0 || heads > 65535 || total_keys < rows || total_keys > 0x7fffff00U) return false;
  for (const void *p : {query, key_cache, value_cache, output})
    if ((reinterpret_cast<std::uintptr_t>(p) & 15U) != 0) return false;
  return true;
}

int flash_tcgen05_attention(const void *query, const void *key_cache, const void *value_cache,
                            const std::size_t rows, const std::size_t total_keys, const std::size_t heads,
                            void *output, cudaStream_t stream) {
  // two CTAs per SM on 64-key tiles (attention_tcgen05_k64.cu) unless EVO_B200_ATTENTION_K64=0 asks for the
  // one-CTA kernel below
  static const bool k64 = [] {
    const char *const flag = std::getenv("EVO_B200_ATTENTION_K64");
    return flag == nullptr || flag[0] != '0';
  }();
  if (k64) return flash_tcgen05_attention_k64(query, key_cache, value_cache, rows, total_keys, heads, output, stream);
  int status = kOk;
  int *const error = error_word(&status, nullptr);
  if (error == nullptr) return status;
  const std::size_t width = heads * kTile;
  CUtensorMap map_q, map_k, map_v;
  if ((status = make_bf16_tile_map(&map_q, query, rows, width, kTile)) != kOk ||
      (status = make_bf16_tile_map(&map_k, key_cache, total_keys, width, kTile)) != kOk ||
      (status = make_bf16_tile_map(&map_v, value_cache, total_keys, width, kTile)) != kOk)
    return status;
  if (cudaFuncSetAttribute(flash_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) !=
      cudaSuccess)
    return fail(kCuda, "cannot raise the attention shared-memory limit");
  const dim3 grid(ceil_div_u(rows, kTile), static_cast<unsigned int>(heads));
  flash_tcgen05_kernel<<<grid, kThreads, kSmemBytes, stream>>>(map_q, map_k, map_v, static_cast<bf16 *>(output),
                                                              static_cast<int>(rows), static_cast<int>(total_keys),
                                                              static_cast<int>(heads), error);
  return check_launch("tcgen05 attention kernel");
}

}  // namespace evob
