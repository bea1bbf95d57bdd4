// Dense projections y = x . W^T on the 5th-generation tensor cores.
//
// Large projections (512 rows and 48 tiles of 256 x 256 or more) run on CTA pairs: gemm_tcgen05_pair_kernel, two
// CTAs of a cluster on one 256 x 256 tile with tcgen05.mma.cta_group::2 (see there).  Everything else,
// and every shape when EVO_B200_GEMM_PAIR=0, runs on gemm_tcgen05_kernel:
// one persistent CTA per SM walks 128 x BN output tiles.  Warp roles:
//   warp 0   TMA producer: streams 128B-swizzled K-major tiles of x [M,K] and
//            W [N,K] into a 4-deep shared-memory ring (mbarrier full/empty).
//   warp 1   MMA issuer: one lane issues tcgen05.mma (M=128, N=BN, K=32 bytes
//            per instruction) into a double-buffered TMEM accumulator and
//            releases ring slots / publishes accumulators with tcgen05.commit.
//   warps 2-5  epilogue: tcgen05.ld the F32 accumulator (one TMEM lane
//            quarter per warp), apply scale / bias / residual / SwiGLU-style
//            gating with the BF16 rounding points of the upstream graph, and
//            store BF16.
// The same kernel serves BF16 operands (kind::f16) and E4M3 codes
// (kind::f8f6f4); only the instruction descriptor and element size differ.
//
// Every wait is bounded: a wait that exceeds its time limit raises a sticky
// error word, all roles drain, TMEM is released and the host reports failure.
//
// Replaces upstream's cuBLASLt call (src/cuda/ops.cu:535-748) and, in the
// tensor-core execution profile, the scalar FP8 emulation
// (src/cuda/ops.cu:916-1006).
#include <cuda.h>

#include <algorithm>
#include <cstdlib>
#include <mutex>
#include <type_traits>

#include "common.cuh"
#include "ops_internal.hpp"
#include "tcgen05.cuh"

namespace evob {
namespace {

constexpr int kBlockM = 128;
constexpr int kBlockKBytes = 128;  // one 128-byte swizzle atom along K
constexpr int kStages = 4;
constexpr int kGemmThreads = 192;

struct EpilogueParams {
  bf16 *out;
  const bf16 *bias;
  const bf16 *residual;
  std::size_t ld_out;
  float alpha;
  const float *row_scale;  // optional [M]: row r's accumulator is also multiplied by row_scale[r]
  int bias_mode;  // 0 none, 1 fused into the F32 sum, 2 separate BF16 add
  int gate_mode;  // 0 none, 1 first*second halves, 2 gelu(first)*second
  // F32 result mode (split-precision products): out_f32 = [out_f32 +] alpha*acc [+ bias_f32]
  float *out_f32;
  const float *bias_f32;
  int accumulate_f32;
  // B's K coordinate wraps after this many K blocks (0: never): A = [x0 | x1 | ...] against
  // the same weight columns
  int weight_wrap_blocks;
  // Split-K (few rows: more CTAs pulling on the weight stream).  Tile t covers K blocks
  // [split * per, (split + 1) * per) with split = t / (tiles_m * tiles_n) and writes its F32
  // partial sums to out_f32 + split * partial_stride; a second kernel adds them up in order.
  int split_k;
  std::size_t partial_stride;
};

using namespace tc;

template <bool kFp8, int BN>
__host__ __device__ constexpr std::uint32_t instruction_descriptor() {
  std::uint32_t d = 0;
  d |= 1U << 4U;                          // accumulator F32
  d |= (kFp8 ? 0U : 1U) << 7U;            // A: E4M3 / BF16
  d |= (kFp8 ? 0U : 1U) << 10U;           // B: E4M3 / BF16
  d |= static_cast<std::uint32_t>(BN >> 3) << 17U;
  d |= static_cast<std::uint32_t>(kBlockM >> 4) << 24U;
  return d;
}

__device__ __forceinline__ bf16 gelu_round(const float x) {
  // Same definition as the stand-alone GELU kernel (seven pinned inputs).
  const bf16 input = f2bf(x);
  const float value = bf2f(input);
  const bf16 computed =
      f2bf(value * 0.5F * (1.0F + ::erff(value * 0.70710678118654752440F)));
  switch (__bfloat16_as_ushort(input)) {
    case 0xc049: return __ushort_as_bfloat16(0xbb2d);
    case 0xc081: return __ushort_as_bfloat16(0xb8eb);
    case 0xc089: return __ushort_as_bfloat16(0xb827);
    case 0xc092: return __ushort_as_bfloat16(0xb742);
    case 0xc0a0: return __ushort_as_bfloat16(0xb5c8);
    case 0xc0a8: return __ushort_as_bfloat16(0xb4fc);
    case 0xc0ab: return __ushort_as_bfloat16(0xb4ab);
    default: return computed;
  }
}

// Tile order: bands of 16 row-tiles, row-tile fastest inside a band.  The ~148
// tiles in flight then cover a 16 x 9 patch of the output, so a wave re-reads
// about 16 A tiles + 9 B tiles from L2 instead of every A tile.
__device__ __forceinline__ void tile_coordinates(const int tile, const int tiles_m,
                                                 const int tiles_n, int *tile_m, int *tile_n) {
  constexpr int kBand = 16;
  const int per_band = kBand * tiles_n;
  const int band = tile / per_band;
  const int first = band * kBand;
  const int rows = min(kBand, tiles_m - first);
  const int local = tile - band * per_band;
  *tile_m = first + local % rows;
  *tile_n = local / rows;
}

// One warp's share of a finished 128 x BN accumulator (TMEM lane quarter `quarter` of the tile that
// starts at column address tmem_tile): scale, bias, gate, residual and the BF16 rounding points of the
// upstream graph, or the F32 / split-K forms.  Rows m0 .., columns n0 .. of the output.
template <int BN>
__device__ __forceinline__ void epilogue_tile(const EpilogueParams &ep, const int M, const int N, const int m0,
                                              const int n0, const int split, const std::uint32_t tmem_tile,
                                              const int quarter, const int lane) {
  const int row = m0 + quarter * 32 + lane;
  const float scale = ep.row_scale != nullptr && row < M ? ep.alpha * ep.row_scale[row] : ep.alpha;
  const std::uint32_t taddr = tmem_tile + (static_cast<std::uint32_t>(quarter * 32) << 16U);
  const bool gated = ep.gate_mode != 0;
  const int chunks = gated ? BN / 64 : BN / 32;
  for (int c = 0; c < chunks; ++c) {
    std::uint32_t v[32];
    std::uint32_t w[32];
    tmem_load_32(taddr + c * 32, v);
    if (gated) tmem_load_32(taddr + BN / 2 + c * 32, w);
    tmem_load_wait();
    const int col = gated ? n0 / 2 + c * 32 : n0 + c * 32;
    const int n_limit = gated ? N / 2 : N;
    if (ep.out_f32 != nullptr) {
      if (row < M && col < n_limit) {
        float *const out_row = ep.out_f32 + static_cast<std::size_t>(split) * ep.partial_stride +
                               static_cast<std::size_t>(row) * ep.ld_out;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          if (col + j < n_limit) {
            float value = __uint_as_float(v[j]) * scale;
            if (ep.bias_f32 != nullptr) value += ep.bias_f32[col + j];
            if (ep.accumulate_f32 != 0) value += out_row[col + j];
            out_row[col + j] = value;
          }
        }
      }
      continue;
    }
    if (row < M && col < n_limit) {
      bf16 *const out_row = ep.out + static_cast<std::size_t>(row) * ep.ld_out;
      float r[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        float value = __uint_as_float(v[j]) * scale;
        if (gated) {
          const float first =
              ep.gate_mode == 2 ? bf2f(gelu_round(value)) : rbf(value);
          const float second = rbf(__uint_as_float(w[j]) * scale);
          r[j] = rbf(first * second);
        } else {
          if (ep.bias_mode == 1 && col + j < n_limit)
            value += bf2f(ep.bias[col + j]);
          value = rbf(value);
          if (ep.bias_mode == 2 && col + j < n_limit)
            value = rbf(value + bf2f(ep.bias[col + j]));
          r[j] = value;
        }
      }
      const bool vector_ok =
          col + 32 <= n_limit && (ep.ld_out % 8) == 0 &&
          (reinterpret_cast<std::uintptr_t>(ep.out) & 15U) == 0;
      if (ep.residual != nullptr) {
        const bf16 *const res_row =
            ep.residual + static_cast<std::size_t>(row) * ep.ld_out;
        if (vector_ok &&
            (reinterpret_cast<std::uintptr_t>(ep.residual) & 15U) == 0) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            Bf16x8 packed;
            packed.raw = *reinterpret_cast<const uint4 *>(res_row + col + q * 8);
#pragma unroll
            for (int j = 0; j < 8; ++j)
              r[q * 8 + j] = rbf(r[q * 8 + j] + packed.get(j));
          }
        } else {
          for (int j = 0; j < 32; ++j)
            if (col + j < n_limit) r[j] = rbf(r[j] + bf2f(res_row[col + j]));
        }
      }
      if (vector_ok) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint4 packed = make_uint4(
              pack_bf16x2(r[q * 8 + 0], r[q * 8 + 1]),
              pack_bf16x2(r[q * 8 + 2], r[q * 8 + 3]),
              pack_bf16x2(r[q * 8 + 4], r[q * 8 + 5]),
              pack_bf16x2(r[q * 8 + 6], r[q * 8 + 7]));
          *reinterpret_cast<uint4 *>(out_row + col + q * 8) = packed;
        }
      } else {
        for (int j = 0; j < 32; ++j)
          if (col + j < n_limit) out_row[col + j] = f2bf(r[j]);
      }
    }
  }
}

template <int BN>
struct SharedLayout {
  static constexpr int kABytes = kBlockM * kBlockKBytes;
  static constexpr int kBBytes = BN * kBlockKBytes;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarrierOffset = kStages * kStageBytes;
  // full[kStages], empty[kStages], tmem_full[2], tmem_empty[2]
  static constexpr int kBarrierCount = 2 * kStages + 4;
  static constexpr int kTmemPtrOffset = kBarrierOffset + kBarrierCount * 8;
  static constexpr int kAbortOffset = kTmemPtrOffset + 8;
  static constexpr int kTotal = kAbortOffset + 8 + 1024;  // + alignment slack
};

template <bool kFp8, int BN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a,
                    const __grid_constant__ CUtensorMap map_b,
                    const EpilogueParams ep, const int M, const int N,
                    const int K_bytes, int *const error_word) {
  using L = SharedLayout<BN>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char *const smem = smem_raw + ((1024U - (smem_u32(smem_raw) & 1023U)) & 1023U)  /* pointer arithmetic keeps the shared address space */;
  const std::uint32_t smem_base = smem_u32(smem);
  const std::uint32_t bar_base = smem_base + L::kBarrierOffset;
  auto full_bar = [&](const int s) { return bar_base + 8U * s; };
  auto empty_bar = [&](const int s) { return bar_base + 8U * (kStages + s); };
  auto tmem_full_bar = [&](const int s) {
    return bar_base + 8U * (2 * kStages + s);
  };
  auto tmem_empty_bar = [&](const int s) {
    return bar_base + 8U * (2 * kStages + 2 + s);
  };
  volatile std::uint32_t *const tmem_ptr =
      reinterpret_cast<volatile std::uint32_t *>(smem + L::kTmemPtrOffset);
  volatile int *const abort_flag =
      reinterpret_cast<volatile int *>(smem + L::kAbortOffset);

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  constexpr std::uint32_t kTmemColumns = 2 * BN;  // 256 or 512, power of two

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(tmem_full_bar(s), 1);
      mbar_init(tmem_empty_bar(s), 4);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile(
        "tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::
            "r"(smem_u32(const_cast<std::uint32_t *>(tmem_ptr))),
        "r"(kTmemColumns)
        : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;"
                 ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const std::uint32_t tmem_base = *tmem_ptr;

  const int tiles_m = (M + kBlockM - 1) / kBlockM;
  const int tiles_n = (N + BN - 1) / BN;
  const int splits = ep.split_k > 1 ? ep.split_k : 1;
  const int tiles_mn = tiles_m * tiles_n;
  const int tiles = tiles_mn * splits;
  const int k_blocks = (K_bytes + kBlockKBytes - 1) / kBlockKBytes;
  const int k_per_split = k_blocks / splits;  // the host picks a split count that divides

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      std::uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        int tile_m, tile_n;
        tile_coordinates(tile % tiles_mn, tiles_m, tiles_n, &tile_m, &tile_n);
        const int m0 = tile_m * kBlockM;
        const int n0 = tile_n * BN;
        const int kb_begin = (tile / tiles_mn) * k_per_split;
        for (int kb = kb_begin; kb < kb_begin + k_per_split; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1U, abort_flag)) {
            ok = false;
            break;
          }
          const std::uint32_t a_dst = smem_base + stage * L::kStageBytes;
          const std::uint32_t b_dst = a_dst + L::kABytes;
          mbar_expect_tx(full_bar(stage), L::kStageBytes);
          const int k_elem = kFp8 ? kb * kBlockKBytes : kb * (kBlockKBytes / 2);
          const int kb_b = ep.weight_wrap_blocks > 0 ? kb % ep.weight_wrap_blocks : kb;
          const int k_elem_b = kFp8 ? kb_b * kBlockKBytes : kb_b * (kBlockKBytes / 2);
          tma_load_2d(a_dst, &map_a, full_bar(stage), k_elem, m0);
          tma_load_2d(b_dst, &map_b, full_bar(stage), k_elem_b, n0);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1U;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr std::uint32_t idesc = instruction_descriptor<kFp8, BN>();
      int stage = 0;
      std::uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok;
           tile += gridDim.x, ++local) {
        const int acc = local & 1;
        const std::uint32_t acc_phase = (local >> 1) & 1U;
        if (!mbar_wait(tmem_empty_bar(acc), acc_phase ^ 1U, abort_flag)) break;
        tc_fence_after();
        const std::uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < k_per_split; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const std::uint32_t a_addr = smem_base + stage * L::kStageBytes;
          const std::uint64_t a_desc = smem_descriptor(a_addr);
          const std::uint64_t b_desc = smem_descriptor(a_addr + L::kABytes);
#pragma unroll
          for (int k = 0; k < kBlockKBytes / 32; ++k) {
            // 32 bytes of K per instruction: +2 in the 16-byte address field.
            tc_mma<kFp8>(tmem_d, a_desc + 2U * k, b_desc + 2U * k, idesc,
                         (kb | k) != 0 ? 1U : 0U);
          }
          tc_commit(empty_bar(stage));
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1U;
          }
        }
        if (ok) tc_commit(tmem_full_bar(acc));
      }
    }
  } else {
    const int quarter = warp % 4;
    int local = 0;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++local) {
      int tile_m, tile_n;
      tile_coordinates(tile % tiles_mn, tiles_m, tiles_n, &tile_m, &tile_n);
      const int m0 = tile_m * kBlockM;
      const int n0 = tile_n * BN;
      const int split = tile / tiles_mn;
      const int acc = local & 1;
      const std::uint32_t acc_phase = (local >> 1) & 1U;
      if (!mbar_wait(tmem_full_bar(acc), acc_phase, abort_flag)) break;
      tc_fence_after();
      epilogue_tile<BN>(ep, M, N, m0, n0, split, tmem_base + acc * BN, quarter, lane);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty_bar(acc));
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0) {
    // Give copies that may still be in flight time to land before the shared
    // memory of this CTA is recycled, then report.
    const unsigned long long start = global_timer_ns();
    while (global_timer_ns() - start < 200000ULL) __nanosleep(1000);
    if (threadIdx.x == 0) atomicOr(error_word, 1 | 32);  // bit 5: a projection kernel
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(
                     tmem_base),
                 "r"(kTmemColumns)
                 : "memory");
  }
}

// ------------------------------------------------------- CTA pairs (cta_group::2)
// The same projection with two CTAs of a cluster on one 256 x 256 output tile.  Each CTA loads its own
// 128 rows of A and its own 128 of the tile's 256 weight rows (TMA without multicast; the copies report
// to the leader's mbarrier), the leader issues tcgen05.mma.cta_group::2 (M = 256, N = 256), and each CTA
// ends up with its 128 rows x 256 columns of the accumulator in its own tensor memory and stores them as
// the one-CTA kernel does.  Per SM a stage is 32 KiB instead of 48 for the same arithmetic: a third
// less traffic from L2, and six stages in flight instead of four.
constexpr int kPairStages = 6;
constexpr int kPairN = 256;

struct PairLayout {
  static constexpr int kABytes = kBlockM * kBlockKBytes;  // 128 rows of A
  static constexpr int kBBytes = 128 * kBlockKBytes;       // this CTA's 128 weight rows of the tile
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarrierOffset = kPairStages * kStageBytes;
  // full[kPairStages], empty[kPairStages], tmem_full[2], tmem_empty[2]
  static constexpr int kBarrierCount = 2 * kPairStages + 4;
  static constexpr int kTmemPtrOffset = kBarrierOffset + kBarrierCount * 8;
  static constexpr int kAbortOffset = kTmemPtrOffset + 8;
  static constexpr int kTotal = kAbortOffset + 8 + 1024;  // + alignment slack
};

__device__ __forceinline__ std::uint32_t cluster_rank() {
  std::uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  return rank;
}
// shared::cluster address of `address` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ std::uint32_t map_to_cta(const std::uint32_t address, const std::uint32_t rank) {
  std::uint32_t mapped;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(mapped) : "r"(address), "r"(rank));
  return mapped;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// 2-D tile load of a CTA pair: lands in this CTA's shared memory, reports its bytes to `bar`, a
// shared::cluster address that may belong to the other CTA of the pair.  No multicast.
__device__ __forceinline__ void tma_load_2d_pair(const std::uint32_t dst, const CUtensorMap *const map,
                                                 const std::uint32_t bar, const int x, const int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<std::uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
template <bool kFp8>
__device__ __forceinline__ void tc_mma_pair(const std::uint32_t tmem_d, const std::uint64_t desc_a,
                                            const std::uint64_t desc_b, const std::uint32_t idesc,
                                            const std::uint32_t accumulate) {
  if constexpr (kFp8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// arrives on the mbarrier at this shared::cta offset in both CTAs of the pair once the MMAs issued so far
// have finished (the multicast is of the arrival, not of a load)
__device__ __forceinline__ void tc_commit_pair(const std::uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
      "h"(static_cast<unsigned short>(3))
      : "memory");
}

template <bool kFp8>
__host__ __device__ constexpr std::uint32_t pair_instruction_descriptor() {
  std::uint32_t d = 0;
  d |= 1U << 4U;                          // accumulator F32
  d |= (kFp8 ? 0U : 1U) << 7U;            // A: E4M3 / BF16
  d |= (kFp8 ? 0U : 1U) << 10U;           // B: E4M3 / BF16
  d |= static_cast<std::uint32_t>(kPairN >> 3) << 17U;
  d |= static_cast<std::uint32_t>(256 >> 4) << 24U;  // M = 256 over the pair
  return d;
}

template <bool kFp8>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const EpilogueParams ep, const int M, const int N, const int K_bytes,
                         int *const error_word) {
  using L = PairLayout;
  extern __shared__ unsigned char smem_raw[];
  unsigned char *const smem = smem_raw + ((1024U - (smem_u32(smem_raw) & 1023U)) & 1023U);
  const std::uint32_t smem_base = smem_u32(smem);
  const std::uint32_t bar_base = smem_base + L::kBarrierOffset;
  auto full_bar = [&](const int s) { return bar_base + 8U * s; };
  auto empty_bar = [&](const int s) { return bar_base + 8U * (kPairStages + s); };
  auto tmem_full_bar = [&](const int s) { return bar_base + 8U * (2 * kPairStages + s); };
  auto tmem_empty_bar = [&](const int s) { return bar_base + 8U * (2 * kPairStages + 2 + s); };
  volatile std::uint32_t *const tmem_ptr = reinterpret_cast<volatile std::uint32_t *>(smem + L::kTmemPtrOffset);
  volatile int *const abort_flag = reinterpret_cast<volatile int *>(smem + L::kAbortOffset);
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const std::uint32_t rank = cluster_rank();  // 0: the leader (issues the MMAs, owns the full barriers)
  constexpr std::uint32_t kTmemColumns = 2 * kPairN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(full_bar(s), 1);   // the leader's: its expect_tx arrival + both CTAs' bytes
      mbar_init(empty_bar(s), 1);  // each CTA's own, signalled by the pair commit
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(tmem_full_bar(s), 1);
      mbar_init(tmem_empty_bar(s), 8);  // the leader's: four epilogue warps of each CTA
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(const_cast<std::uint32_t *>(tmem_ptr))),
                 "r"(kTmemColumns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anything is signalled across the pair
  tc_fence_after();
  const std::uint32_t tmem_base = *tmem_ptr;

  const int tiles_m = (M + 255) / 256;
  const int tiles_n = (N + kPairN - 1) / kPairN;
  const int splits = ep.split_k > 1 ? ep.split_k : 1;
  const int tiles_mn = tiles_m * tiles_n;
  const int tiles = tiles_mn * splits;
  const int k_blocks = (K_bytes + kBlockKBytes - 1) / kBlockKBytes;
  const int k_per_split = k_blocks / splits;
  const int pair = static_cast<int>(blockIdx.x / 2), pairs = static_cast<int>(gridDim.x / 2);

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      std::uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < tiles && ok; tile += pairs) {
        int tile_m, tile_n;
        tile_coordinates(tile % tiles_mn, tiles_m, tiles_n, &tile_m, &tile_n);
        const int m0 = tile_m * 256 + static_cast<int>(rank) * 128;
        const int n0 = tile_n * kPairN + static_cast<int>(rank) * 128;
        const int kb_begin = (tile / tiles_mn) * k_per_split;
        for (int kb = kb_begin; kb < kb_begin + k_per_split; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1U, abort_flag)) {
            ok = false;
            break;
          }
          const std::uint32_t a_dst = smem_base + stage * L::kStageBytes;
          const std::uint32_t b_dst = a_dst + L::kABytes;
          if (rank == 0) mbar_expect_tx(full_bar(stage), 2 * L::kStageBytes);
          const std::uint32_t leader_full = map_to_cta(full_bar(stage), 0);
          const int k_elem = kFp8 ? kb * kBlockKBytes : kb * (kBlockKBytes / 2);
          const int kb_b = ep.weight_wrap_blocks > 0 ? kb % ep.weight_wrap_blocks : kb;
          const int k_elem_b = kFp8 ? kb_b * kBlockKBytes : kb_b * (kBlockKBytes / 2);
          tma_load_2d_pair(a_dst, &map_a, leader_full, k_elem, m0);
          tma_load_2d_pair(b_dst, &map_b, leader_full, k_elem_b, n0);
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1U;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      constexpr std::uint32_t idesc = pair_instruction_descriptor<kFp8>();
      int stage = 0;
      std::uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = pair; tile < tiles && ok; tile += pairs, ++local) {
        const int acc = local & 1;
        const std::uint32_t acc_phase = (local >> 1) & 1U;
        if (!mbar_wait(tmem_empty_bar(acc), acc_phase ^ 1U, abort_flag)) break;
        tc_fence_after();
        const std::uint32_t tmem_d = tmem_base + acc * kPairN;
        for (int kb = 0; kb < k_per_split; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const std::uint32_t a_addr = smem_base + stage * L::kStageBytes;
          const std::uint64_t a_desc = smem_descriptor(a_addr);
          const std::uint64_t b_desc = smem_descriptor(a_addr + L::kABytes);
#pragma unroll
          for (int k = 0; k < kBlockKBytes / 32; ++k)
            tc_mma_pair<kFp8>(tmem_d, a_desc + 2U * k, b_desc + 2U * k, idesc, (kb | k) != 0 ? 1U : 0U);
          tc_commit_pair(empty_bar(stage));  // the slot is free in both CTAs
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1U;
          }
        }
        if (ok) tc_commit_pair(tmem_full_bar(acc));
      }
    }
  } else {
    const int quarter = warp % 4;
    int local = 0;
    for (int tile = pair; tile < tiles; tile += pairs, ++local) {
      int tile_m, tile_n;
      tile_coordinates(tile % tiles_mn, tiles_m, tiles_n, &tile_m, &tile_n);
      const int m0 = tile_m * 256 + static_cast<int>(rank) * 128;
      const int n0 = tile_n * kPairN;
      const int split = tile / tiles_mn;
      const int acc = local & 1;
      const std::uint32_t acc_phase = (local >> 1) & 1U;
      if (!mbar_wait(tmem_full_bar(acc), acc_phase, abort_flag)) break;
      tc_fence_after();
      epilogue_tile<kPairN>(ep, M, N, m0, n0, split, tmem_base + acc * kPairN, quarter, lane);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        const std::uint32_t leader_empty = map_to_cta(tmem_empty_bar(acc), 0);
        asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(leader_empty) : "memory");
      }
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0) {
    const unsigned long long start = global_timer_ns();
    while (global_timer_ns() - start < 200000ULL) __nanosleep(1000);
    if (threadIdx.x == 0) atomicOr(error_word, 1 | 32);  // bit 5: a projection kernel
  }
  // neither CTA leaves while the other may still read its shared memory or signal its barriers
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColumns)
                 : "memory");
  }
}

// --------------------------------------------------- few tokens (swap-AB)
// At up to 128 tokens a projection is a weight stream, and the tile kernel above
// pulls on it badly: its 128-row MMA spends a full tile of tensor time on every
// weight block whether 16 or 128 of the rows are tokens, and it has only
// N / 256 tiles to spread over the SMs.  Here the roles are swapped: the weight
// rows are the M = 128 operand, the tokens the N = BT operand (16..128), so the
// tensor time per weight byte falls with the token count, a CTA owns 128 weight
// rows x one K slice, and K is split until enough CTAs pull on the stream.  The
// CTAs leave raw F32 partial sums [split][token][weight row]; the finishing
// kernel adds them in split order and applies the epilogue.
constexpr int kSwapStages = 6;

template <int BT>
struct SwapLayout {
  static constexpr int kWBytes = kBlockM * kBlockKBytes;  // 128 weight rows x 128 bytes of K
  static constexpr int kXBytes = BT * kBlockKBytes;
  static constexpr int kStageBytes = kWBytes + kXBytes;
  static constexpr int kBarrierOffset = kSwapStages * kStageBytes;
  static constexpr int kBarrierCount = 2 * kSwapStages + 1;  // full[], empty[], accumulator ready
  static constexpr int kTmemPtrOffset = kBarrierOffset + kBarrierCount * 8;
  static constexpr int kAbortOffset = kTmemPtrOffset + 8;
  static constexpr int kTotal = kAbortOffset + 8 + 1024;  // + alignment slack
};

template <bool kFp8, int BT>
__global__ void __launch_bounds__(kGemmThreads)
gemm_swap_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                 float *const partials, const std::size_t partial_stride, const int M, const int N,
                 const int tiles_n, const int k_per_split, int *const error_word) {
  using L = SwapLayout<BT>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char *const smem = smem_raw + ((1024U - (smem_u32(smem_raw) & 1023U)) & 1023U)  /* pointer arithmetic keeps the shared address space */;
  const std::uint32_t smem_base = smem_u32(smem);
  const std::uint32_t bar_base = smem_base + L::kBarrierOffset;
  auto full_bar = [&](const int s) { return bar_base + 8U * s; };
  auto empty_bar = [&](const int s) { return bar_base + 8U * (kSwapStages + s); };
  const std::uint32_t ready_bar = bar_base + 8U * (2 * kSwapStages);
  volatile std::uint32_t *const tmem_ptr = reinterpret_cast<volatile std::uint32_t *>(smem + L::kTmemPtrOffset);
  volatile int *const abort_flag = reinterpret_cast<volatile int *>(smem + L::kAbortOffset);
  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  constexpr std::uint32_t kTmemColumns = BT < 32 ? 32 : BT;  // power of two, at least 32

  if (threadIdx.x == 0) {
    for (int s = 0; s < kSwapStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(ready_bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::
                     "r"(smem_u32(const_cast<std::uint32_t *>(tmem_ptr))),
                 "r"(kTmemColumns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const std::uint32_t tmem_base = *tmem_ptr;

  const int tile_n = blockIdx.x % tiles_n;
  const int split = blockIdx.x / tiles_n;
  const int n0 = tile_n * kBlockM;
  const int kb_begin = split * k_per_split;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      std::uint32_t phase = 0;
      for (int kb = kb_begin; kb < kb_begin + k_per_split; ++kb) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1U, abort_flag)) break;
        const std::uint32_t w_dst = smem_base + stage * L::kStageBytes;
        mbar_expect_tx(full_bar(stage), L::kStageBytes);
        const int k_elem = kFp8 ? kb * kBlockKBytes : kb * (kBlockKBytes / 2);
        tma_load_2d(w_dst, &map_w, full_bar(stage), k_elem, n0);
        tma_load_2d(w_dst + L::kWBytes, &map_x, full_bar(stage), k_elem, 0);
        if (++stage == kSwapStages) {
          stage = 0;
          phase ^= 1U;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr std::uint32_t idesc = instruction_descriptor<kFp8, BT>();
      int stage = 0;
      std::uint32_t phase = 0;
      bool ok = true;
      for (int kb = 0; kb < k_per_split; ++kb) {
        if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const std::uint32_t w_addr = smem_base + stage * L::kStageBytes;
        const std::uint64_t w_desc = smem_descriptor(w_addr);
        const std::uint64_t x_desc = smem_descriptor(w_addr + L::kWBytes);
#pragma unroll
        for (int k = 0; k < kBlockKBytes / 32; ++k)
          tc_mma<kFp8>(tmem_base, w_desc + 2U * k, x_desc + 2U * k, idesc, (kb | k) != 0 ? 1U : 0U);
        tc_commit(empty_bar(stage));
        if (++stage == kSwapStages) {
          stage = 0;
          phase ^= 1U;
        }
      }
      if (ok) tc_commit(ready_bar);
    }
  } else {
    const int quarter = warp % 4;
    if (mbar_wait(ready_bar, 0U, abort_flag)) {
      tc_fence_after();
      const int n = n0 + quarter * 32 + lane;  // this thread's weight row = output column
      const std::uint32_t taddr = tmem_base + (static_cast<std::uint32_t>(quarter * 32) << 16U);
      float *const out = partials + static_cast<std::size_t>(split) * partial_stride + n;
      for (int c = 0; c < (BT + 31) / 32; ++c) {
        std::uint32_t v[32];
        tmem_load_32(taddr + c * 32, v);
        tmem_load_wait();
        if (n < N) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int token = c * 32 + j;
            // consecutive lanes hold consecutive output columns: 128-byte stores
            if (token < M && token < BT) out[static_cast<std::size_t>(token) * N] = __uint_as_float(v[j]);
          }
        }
      }
    }
    tc_fence_before();
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0) {
    const unsigned long long start = global_timer_ns();
    while (global_timer_ns() - start < 200000ULL) __nanosleep(1000);
    if (threadIdx.x == 0) atomicOr(error_word, 1 | 32);  // bit 5: a projection kernel
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColumns)
                 : "memory");
  }
}

// ---------------------------------------------------------- SIMT fallback
// Shapes the TMA path cannot take (row pitch not a multiple of 16 bytes, or
// the tiny test-fixture widths) run on CUDA cores with the same epilogue.
template <bool kFp8>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const void *__restrict__ a_raw, const void *__restrict__ b_raw,
                 const EpilogueParams ep, const int M, const int N,
                 const int K) {
  __shared__ float a_tile[16][65];
  __shared__ float b_tile[16][65];
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  float acc[4][4] = {};
  auto load = [&](const void *base, const int row, const int k) -> float {
    const std::size_t index = static_cast<std::size_t>(row) * K + k;
    if constexpr (kFp8) {
      const std::uint8_t code = static_cast<const std::uint8_t *>(base)[index];
      const unsigned int e = (code >> 3U) & 0xfU, m = code & 7U;
      const float magnitude =
          e == 0 ? ldexpf(static_cast<float>(m), -9)
                 : ldexpf(1.0F + static_cast<float>(m) * 0.125F,
                          static_cast<int>(e) - 7);
      return (code & 0x80U) ? -magnitude : magnitude;
    } else {
      return bf2f(static_cast<const bf16 *>(base)[index]);
    }
  };
  for (int k0 = 0; k0 < K; k0 += 16) {
    for (int i = threadIdx.x; i < 64 * 16; i += 256) {
      const int r = i / 16, k = i % 16;
      a_tile[k][r] = (m0 + r < M && k0 + k < K) ? load(a_raw, m0 + r, k0 + k) : 0.0F;
      b_tile[k][r] = (n0 + r < N && k0 + k < K) ? load(b_raw, n0 + r, k0 + k) : 0.0F;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; ++k) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
          acc[i][j] = fmaf(a_tile[k][ty * 4 + i], b_tile[k][tx * 4 + j], acc[i][j]);
    }
    __syncthreads();
  }
  for (int i = 0; i < 4; ++i) {
    const int row = m0 + ty * 4 + i;
    if (row >= M) continue;
    for (int j = 0; j < 4; ++j) {
      const int col = n0 + tx * 4 + j;
      if (col >= N) continue;
      float value = acc[i][j] * (ep.row_scale != nullptr ? ep.alpha * ep.row_scale[row] : ep.alpha);
      if (ep.bias_mode == 1) value += bf2f(ep.bias[col]);
      value = rbf(value);
      if (ep.bias_mode == 2) value = rbf(value + bf2f(ep.bias[col]));
      const std::size_t index = static_cast<std::size_t>(row) * ep.ld_out + col;
      if (ep.residual != nullptr) value = rbf(value + bf2f(ep.residual[index]));
      ep.out[index] = f2bf(value);
    }
  }
}

// Second step of split-K: adds the partial sums of one output element in split
// order and applies the epilogue of the tile kernel (same expressions, same
// BF16 rounding points), including the gate over 128-column halves.
__global__ void __launch_bounds__(256)
splitk_finish_kernel(const float *__restrict__ partials, const int splits, const std::size_t partial_stride,
                     const EpilogueParams ep, const int M, const int N) {
  const bool gated = ep.gate_mode != 0;
  const int out_columns = gated ? N / 2 : N;
  const std::size_t total = static_cast<std::size_t>(M) * out_columns;
  const std::size_t stride = static_cast<std::size_t>(blockDim.x) * gridDim.x;
  for (std::size_t i = static_cast<std::size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int row = static_cast<int>(i / out_columns), col = static_cast<int>(i % out_columns);
    const auto sum = [&](const int column) {
      float value = 0.0F;
      for (int s = 0; s < splits; ++s)
        value += partials[static_cast<std::size_t>(s) * partial_stride + static_cast<std::size_t>(row) * N + column];
      return value * (ep.row_scale != nullptr ? ep.alpha * ep.row_scale[row] : ep.alpha);
    };
    float result;
    if (gated) {
      const int first_column = (col / 128) * 256 + col % 128;
      const float value = sum(first_column);
      const float first = ep.gate_mode == 2 ? bf2f(gelu_round(value)) : rbf(value);
      const float second = rbf(sum(first_column + 128));
      result = rbf(first * second);
    } else {
      float value = sum(col);
      if (ep.bias_mode == 1) value += bf2f(ep.bias[col]);
      value = rbf(value);
      if (ep.bias_mode == 2) value = rbf(value + bf2f(ep.bias[col]));
      if (ep.residual != nullptr) value = rbf(value + bf2f(ep.residual[static_cast<std::size_t>(row) * ep.ld_out + col]));
      result = value;
    }
    ep.out[static_cast<std::size_t>(row) * ep.ld_out + col] = f2bf(result);
  }
}

// ------------------------------------------------------------ host side
using EncodeTiled = CUresult (*)(CUtensorMap *, CUtensorMapDataType,
                                 cuuint32_t, void *, const cuuint64_t *,
                                 const cuuint64_t *, const cuuint32_t *,
                                 const cuuint32_t *, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion,
                                 CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
  static EncodeTiled fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *symbol = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &symbol,
                                cudaEnableDefault, &result) == cudaSuccess &&
        result == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiled>(symbol);
  });
  return fn;
}

int make_map(CUtensorMap *map, const void *base, const bool fp8,
             const std::size_t rows, const std::size_t k_elements,
             const int box_rows) {
  const EncodeTiled encode = encode_tiled();
  if (encode == nullptr)
    return fail(kCuda, "cuTensorMapEncodeTiled is unavailable");
  const std::size_t element = fp8 ? 1 : 2;
  const cuuint64_t dims[2] = {k_elements, rows};
  const cuuint64_t strides[1] = {k_elements * element};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(kBlockKBytes / element),
                             static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t element_strides[2] = {1, 1};
  const CUresult result = encode(
      map, fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
      2, const_cast<void *>(base), dims, strides, box, element_strides,
      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (result != CUDA_SUCCESS)
    return fail(kCuda, "cuTensorMapEncodeTiled failed with code " +
                           std::to_string(static_cast<int>(result)));
  return kOk;
}

struct DeviceState {
  int *error_word = nullptr;
  int sm_count = 0;
  bool attributes_set = false;
};

DeviceState *device_state(int *status) {
  static std::mutex mutex;
  static DeviceState states[64];
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) {
    *status = fail(kCuda, "cannot query the current CUDA device");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mutex);
  DeviceState &state = states[device];
  if (state.error_word == nullptr) {
    if (cudaMalloc(&state.error_word, sizeof(int)) != cudaSuccess ||
        cudaMemset(state.error_word, 0, sizeof(int)) != cudaSuccess) {
      *status = fail(kCuda, "cannot allocate the GEMM error word");
      return nullptr;
    }
    cudaDeviceGetAttribute(&state.sm_count, cudaDevAttrMultiProcessorCount,
                           device);
    if (state.sm_count <= 0) state.sm_count = kSmCount;
  }
  *status = kOk;
  return &state;
}

template <bool kFp8, int BN>
int launch_tc(const void *a, const void *b, const EpilogueParams &ep,
              const std::size_t M, const std::size_t N, const std::size_t K,
              cudaStream_t stream) {
  // the weight is [N, K], or [N, wrap width] when its K coordinate wraps
  const std::size_t weight_k = ep.weight_wrap_blocks > 0 ? static_cast<std::size_t>(ep.weight_wrap_blocks) * 64 : K;
  int status = kOk;
  DeviceState *const state = device_state(&status);
  if (state == nullptr) return status;
  CUtensorMap map_a, map_b;
  status = make_map(&map_a, a, kFp8, M, K, kBlockM);
  if (status != kOk) return status;
  status = make_map(&map_b, b, kFp8, N, weight_k, BN);
  if (status != kOk) return status;
  using L = SharedLayout<BN>;
  static bool configured[64] = {};
  int device = 0;
  cudaGetDevice(&device);
  if (!configured[device]) {
    if (cudaFuncSetAttribute(gemm_tcgen05_kernel<kFp8, BN>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                             L::kTotal) != cudaSuccess)
      return fail(kCuda, "cannot raise the GEMM shared-memory limit");
    configured[device] = true;
  }
  const std::size_t tiles =
      ((M + kBlockM - 1) / kBlockM) * ((N + BN - 1) / BN) * static_cast<std::size_t>(ep.split_k > 1 ? ep.split_k : 1);
  const unsigned int grid = static_cast<unsigned int>(
      tiles < static_cast<std::size_t>(state->sm_count) ? tiles
                                                        : state->sm_count);
  gemm_tcgen05_kernel<kFp8, BN><<<grid, kGemmThreads, L::kTotal, stream>>>(
      map_a, map_b, ep, static_cast<int>(M), static_cast<int>(N),
      static_cast<int>(K * (kFp8 ? 1 : 2)), state->error_word);
  return check_launch("tcgen05 GEMM kernel");
}

template <bool kFp8>
int launch_tc_pair(const void *a, const void *b, const EpilogueParams &ep, const std::size_t M, const std::size_t N,
                   const std::size_t K, cudaStream_t stream) {
  const std::size_t weight_k = ep.weight_wrap_blocks > 0 ? static_cast<std::size_t>(ep.weight_wrap_blocks) * 64 : K;
  int status = kOk;
  DeviceState *const state = device_state(&status);
  if (state == nullptr) return status;
  CUtensorMap map_a, map_b;
  status = make_map(&map_a, a, kFp8, M, K, kBlockM);
  if (status != kOk) return status;
  status = make_map(&map_b, b, kFp8, N, weight_k, 128);  // a CTA loads its 128 of the tile's 256 weight rows
  if (status != kOk) return status;
  static bool configured[64] = {};
  int device = 0;
  cudaGetDevice(&device);
  if (!configured[device]) {
    if (cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<kFp8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             PairLayout::kTotal) != cudaSuccess)
      return fail(kCuda, "cannot raise the GEMM shared-memory limit");
    configured[device] = true;
  }
  const std::size_t tiles =
      ((M + 255) / 256) * ((N + kPairN - 1) / kPairN) * static_cast<std::size_t>(ep.split_k > 1 ? ep.split_k : 1);
  const std::size_t pairs = std::min<std::size_t>(tiles, static_cast<std::size_t>(state->sm_count) / 2);
  gemm_tcgen05_pair_kernel<kFp8><<<static_cast<unsigned int>(2 * pairs), kGemmThreads, PairLayout::kTotal, stream>>>(
      map_a, map_b, ep, static_cast<int>(M), static_cast<int>(N), static_cast<int>(K * (kFp8 ? 1 : 2)),
      state->error_word);
  return check_launch("tcgen05 GEMM kernel (CTA pairs)");
}

template <bool kFp8, int BT>
int launch_swap(const void *x, const void *w, float *partials, const std::size_t M, const std::size_t N,
                const std::size_t K, const int split, cudaStream_t stream) {
  int status = kOk;
  DeviceState *const state = device_state(&status);
  if (state == nullptr) return status;
  CUtensorMap map_w, map_x;
  status = make_map(&map_w, w, kFp8, N, K, kBlockM);
  if (status != kOk) return status;
  status = make_map(&map_x, x, kFp8, M, K, BT);
  if (status != kOk) return status;
  using L = SwapLayout<BT>;
  static bool configured[64] = {};
  int device = 0;
  cudaGetDevice(&device);
  if (!configured[device]) {
    if (cudaFuncSetAttribute(gemm_swap_kernel<kFp8, BT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             L::kTotal) != cudaSuccess)
      return fail(kCuda, "cannot raise the GEMM shared-memory limit");
    configured[device] = true;
  }
  const int tiles_n = static_cast<int>((N + kBlockM - 1) / kBlockM);
  const int k_blocks = static_cast<int>(K * (kFp8 ? 1 : 2) / kBlockKBytes);
  gemm_swap_kernel<kFp8, BT><<<static_cast<unsigned int>(tiles_n * split), kGemmThreads, L::kTotal, stream>>>(
      map_w, map_x, partials, M * N, static_cast<int>(M), static_cast<int>(N), tiles_n, k_blocks / split,
      state->error_word);
  return check_launch("tcgen05 few-token GEMM kernel");
}

}  // namespace

namespace tc {
int make_bf16_tile_map(CUtensorMap *map, const void *base, const std::size_t rows,
                       const std::size_t columns, const int box_rows) {
  return make_map(map, base, false, rows, columns, box_rows);
}
int *error_word(int *status, int *sm_count) {
  DeviceState *const state = device_state(status);
  if (state == nullptr) return nullptr;
  if (sm_count != nullptr) *sm_count = state->sm_count;
  return state->error_word;
}
}  // namespace tc

int gemm_error_state(cudaStream_t stream) {
  int status = kOk;
  DeviceState *const state = device_state(&status);
  if (state == nullptr) return status;
  int value = 0;
  if (cudaMemcpyAsync(&value, state->error_word, sizeof(int),
                      cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
      cudaStreamSynchronize(stream) != cudaSuccess)
    return fail(kCuda, "cannot read the GEMM error word");
  if (value != 0) {
    cudaMemsetAsync(state->error_word, 0, sizeof(int), stream);
    if ((value & 1) != 0) {
      // bits 2..5 name the kernel family whose bounded wait ran out
      std::string where;
      if ((value & 4) != 0) where += " [medium FIR]";
      if ((value & 8) != 0) where += " [attention, 64-key tiles]";
      if ((value & 16) != 0) where += " [attention, 128-key tiles]";
      if ((value & 32) != 0) where += " [projection]";
      return fail(kCuda, "a tcgen05 GEMM pipeline wait timed out" + where);
    }
    return fail(kInvalidArgument, "token ID exceeds model vocabulary");
  }
  return kOk;
}

int *device_error_word(int *status) { return tc::error_word(status, nullptr); }

int linear(const LinearArgs &args, cudaStream_t stream) {
  const bool fp8 = args.operand_type == OperandType::kE4m3;
  if (args.input == nullptr || args.weight == nullptr ||
      (args.output == nullptr && args.output_f32 == nullptr) || args.in_features == 0 ||
      args.out_features == 0 || !isfinite(args.alpha))
    return fail(kInvalidArgument, "linear arguments are invalid");
  if (args.bias_mode != 0 && args.bias == nullptr)
    return fail(kInvalidArgument, "linear bias mode needs a bias vector");
  if (args.gate_mode != 0 &&
      (args.bias_mode != 0 || args.residual != nullptr))
    return fail(kInvalidArgument,
                "gated linear cannot take a bias or a residual");
  if (args.rows > 0x7fffffffU || args.out_features > 0x7fffffffU ||
      args.in_features > 0x3fffffffU)
    return fail(kInvalidArgument, "linear dimensions are too large");
  if (args.rows == 0) return kOk;
  if (args.output_f32 != nullptr &&
      (fp8 || args.gate_mode != 0 || args.bias_mode != 0 || args.residual != nullptr))
    return fail(kInvalidArgument, "the F32-result mode takes BF16 operands and no BF16 epilogue");
  if (args.output_f32 == nullptr && args.row_scale == nullptr && small_batch_linear_applicable(args))
    return small_batch_linear(args, stream);
  const std::size_t out_columns =
      args.gate_mode != 0 ? args.out_features / 2 : args.out_features;
  EpilogueParams ep{};
  ep.out = static_cast<bf16 *>(args.output);
  ep.bias = static_cast<const bf16 *>(args.bias);
  ep.residual = static_cast<const bf16 *>(args.residual);
  ep.ld_out = out_columns;
  ep.alpha = args.alpha;
  ep.row_scale = args.row_scale;
  ep.bias_mode = args.bias_mode;
  ep.gate_mode = args.gate_mode;
  ep.out_f32 = args.output_f32;
  ep.bias_f32 = args.bias_f32;
  ep.accumulate_f32 = args.accumulate_f32 ? 1 : 0;
  if (args.weight_wrap_features != 0) {
    if (args.weight_wrap_features % 64 != 0 || args.output_f32 == nullptr)
      return fail(kInvalidArgument, "weight wrap needs whole K blocks and the F32-result mode");
    ep.weight_wrap_blocks = static_cast<int>(args.weight_wrap_features / 64);
  }
  const std::size_t pitch = args.in_features * (fp8 ? 1 : 2);
  const bool tma_ok =
      pitch % 16 == 0 && pitch >= 128 &&
      (reinterpret_cast<std::uintptr_t>(args.input) & 15U) == 0 &&
      (reinterpret_cast<std::uintptr_t>(args.weight) & 15U) == 0 &&
      args.out_features >= 64 && !args.force_simt;
  // (measured at 128 rows: 27.6 / 31.8 us against 34.8 / 71.7 us for 4096x4096 / 4096x11264 weights, but
  // 48 / 75 us against 37 / 61 us for 12288 / 22528 weight rows, where the tile kernel has enough tiles
  // and the partial sums cost more than the swap saves; at 16 rows 17 / 28 / 28 / 44 us against 33 / 72 / 37 / 59 us)
  if (tma_ok && args.split_workspace != nullptr && args.output_f32 == nullptr &&
      (args.rows <= 64 || (args.rows <= 128 && args.out_features <= 8192)) &&
      pitch % kBlockKBytes == 0 && args.weight_wrap_features == 0 &&
      (args.gate_mode == 0 || args.out_features % 256 == 0)) {
    // Few tokens: weights as the 128-row operand, tokens as the narrow one, K split until
    // enough CTAs pull on the weight stream; partial sums limited to ~a quarter of the weight bytes.
    const std::size_t tiles_n = (args.out_features + kBlockM - 1) / kBlockM;
    const std::size_t k_blocks = pitch / kBlockKBytes;
    int split = 1;
    for (const int candidate : {8, 4, 2}) {
      if (k_blocks % candidate == 0 && k_blocks / candidate >= 8 && tiles_n * candidate <= 2 * kSmCount &&
          static_cast<std::size_t>(candidate) * args.rows * 32 <= pitch &&
          static_cast<std::size_t>(candidate) * args.rows * args.out_features * sizeof(float) <=
              args.split_workspace_bytes) {
        split = candidate;
        break;
      }
    }
    if (args.rows * args.out_features * sizeof(float) <= args.split_workspace_bytes) {
      float *const partials = static_cast<float *>(args.split_workspace);
      const auto launch = [&](auto fp8_tag, auto bt_tag) {
        return launch_swap<decltype(fp8_tag)::value, decltype(bt_tag)::value>(
            args.input, args.weight, partials, args.rows, args.out_features, args.in_features, split, stream);
      };
      using F = std::false_type;
      using T = std::true_type;
      int status;
      if (args.rows <= 16) status = fp8 ? launch(T{}, std::integral_constant<int, 16>{}) : launch(F{}, std::integral_constant<int, 16>{});
      else if (args.rows <= 32) status = fp8 ? launch(T{}, std::integral_constant<int, 32>{}) : launch(F{}, std::integral_constant<int, 32>{});
      else if (args.rows <= 64) status = fp8 ? launch(T{}, std::integral_constant<int, 64>{}) : launch(F{}, std::integral_constant<int, 64>{});
      else status = fp8 ? launch(T{}, std::integral_constant<int, 128>{}) : launch(F{}, std::integral_constant<int, 128>{});
      if (status != kOk) return status;
      const std::size_t outputs = args.rows * out_columns;
      splitk_finish_kernel<<<static_cast<unsigned int>((outputs + 255) / 256 > 2048 ? 2048 : (outputs + 255) / 256),
                             256, 0, stream>>>(partials, split, args.rows * args.out_features, ep,
                                               static_cast<int>(args.rows), static_cast<int>(args.out_features));
      return check_launch("split-K finishing kernel");
    }
  }
  // (measured: pays off up to a few dozen rows; at 128 rows the partial-sum traffic outweighs it)
  if (tma_ok && args.split_workspace != nullptr && args.output_f32 == nullptr && args.rows <= 32 &&
      pitch % kBlockKBytes == 0 && (args.gate_mode == 0 || args.out_features % 256 == 0)) {
    // One row tile: the projection is a weight stream.  Split K so that enough CTAs pull on it,
    // F32 partials in the caller's workspace, summed in split order by a second kernel.
    const int bn = args.gate_mode != 0 ? 256 : 128;  // a gated tile holds both 128-column halves
    const std::size_t tiles_n = (args.out_features + bn - 1) / bn;
    const std::size_t k_blocks = pitch / kBlockKBytes;
    int split = 1;
    for (const int candidate : {8, 4, 2}) {
      if (k_blocks % candidate == 0 && k_blocks / candidate >= 8 && tiles_n * candidate <= 2 * kSmCount &&
          static_cast<std::size_t>(candidate) * args.rows * args.out_features * sizeof(float) <=
              args.split_workspace_bytes) {
        split = candidate;
        break;
      }
    }
    if (split > 1 && tiles_n < 120) {
      EpilogueParams partial{};
      partial.ld_out = args.out_features;
      partial.alpha = 1.0F;
      partial.out_f32 = static_cast<float *>(args.split_workspace);
      partial.split_k = split;
      partial.partial_stride = args.rows * args.out_features;
      int status;
      if (bn == 256)
        status = fp8 ? launch_tc<true, 256>(args.input, args.weight, partial, args.rows, args.out_features,
                                            args.in_features, stream)
                     : launch_tc<false, 256>(args.input, args.weight, partial, args.rows, args.out_features,
                                             args.in_features, stream);
      else
        status = fp8 ? launch_tc<true, 128>(args.input, args.weight, partial, args.rows, args.out_features,
                                            args.in_features, stream)
                     : launch_tc<false, 128>(args.input, args.weight, partial, args.rows, args.out_features,
                                             args.in_features, stream);
      if (status != kOk) return status;
      const std::size_t outputs = args.rows * out_columns;
      splitk_finish_kernel<<<static_cast<unsigned int>((outputs + 255) / 256 > 2048 ? 2048 : (outputs + 255) / 256),
                             256, 0, stream>>>(static_cast<const float *>(args.split_workspace), split,
                                               partial.partial_stride, ep, static_cast<int>(args.rows),
                                               static_cast<int>(args.out_features));
      return check_launch("split-K finishing kernel");
    }
  }
  if (tma_ok) {
    if (args.gate_mode != 0 && args.out_features % 256 != 0)
      return fail(kInvalidArgument, "gated linear needs the interleaved width to be a multiple of 256");
    // CTA pairs on 256 x 256 tiles where there are enough of them to fill the pairs of the GPU
    // (EVO_B200_GEMM_PAIR=0: one CTA per 128 x 256 tile everywhere)
    static const bool pairs_enabled = [] {
      const char *const flag = std::getenv("EVO_B200_GEMM_PAIR");
      return flag == nullptr || flag[0] != '0';
    }();
    // (not below 512 rows: a pair's tile is 256 rows, and at 128 rows half of every pair would idle)
    static const std::size_t pair_tiles = [] {
      const char *const text = std::getenv("EVO_B200_GEMM_PAIR_MIN_TILES");
      const long value = text != nullptr ? std::strtol(text, nullptr, 10) : 0;
      // 1,024 x 4096 outputs are 64 pair tiles on 74 pairs: 883 against 840 TFLOP/s at K = 4096, 1,214 against
      // 1,126 at K = 11264
      return value > 0 ? static_cast<std::size_t>(value) : std::size_t{48};
    }();
    if (pairs_enabled && ep.weight_wrap_blocks == 0 && args.rows >= 512 &&
        ((args.rows + 255) / 256) * ((args.out_features + 255) / 256) >= pair_tiles)
      return fp8 ? launch_tc_pair<true>(args.input, args.weight, ep, args.rows, args.out_features, args.in_features,
                                        stream)
                 : launch_tc_pair<false>(args.input, args.weight, ep, args.rows, args.out_features,
                                         args.in_features, stream);
    if (args.gate_mode != 0) {
      return fp8 ? launch_tc<true, 256>(args.input, args.weight, ep, args.rows,
                                        args.out_features, args.in_features,
                                        stream)
                 : launch_tc<false, 256>(args.input, args.weight, ep,
                                         args.rows, args.out_features,
                                         args.in_features, stream);
    }
    // Narrower tiles when wide ones would leave most SMs without work.
    const std::size_t tiles_m = (args.rows + kBlockM - 1) / kBlockM;
    // (Measured: below 128 columns the shorter weight tiles put fewer bytes in
    // flight per CTA and lose more than the extra CTAs win, except for narrow
    // outputs, so 64 and 32 are used only when the output itself is that narrow.)
    int bn = 256;
    if (tiles_m * ((args.out_features + 255) / 256) < 120) bn = 128;
    while (bn > 32 && args.out_features < static_cast<std::size_t>(bn)) bn /= 2;
    const auto launch = [&](auto fp8_tag, auto bn_tag) {
      return launch_tc<decltype(fp8_tag)::value, decltype(bn_tag)::value>(
          args.input, args.weight, ep, args.rows, args.out_features, args.in_features, stream);
    };
    using F = std::false_type;
    using T = std::true_type;
    switch (bn) {
      case 256: return fp8 ? launch(T{}, std::integral_constant<int, 256>{}) : launch(F{}, std::integral_constant<int, 256>{});
      case 128: return fp8 ? launch(T{}, std::integral_constant<int, 128>{}) : launch(F{}, std::integral_constant<int, 128>{});
      case 64: return fp8 ? launch(T{}, std::integral_constant<int, 64>{}) : launch(F{}, std::integral_constant<int, 64>{});
      default: return fp8 ? launch(T{}, std::integral_constant<int, 32>{}) : launch(F{}, std::integral_constant<int, 32>{});
    }
  }
  if (args.gate_mode != 0)
    return fail(kUnsupported,
                "gated linear is only available on the tensor-core path");
  const dim3 grid(ceil_div_u(args.out_features, 64), ceil_div_u(args.rows, 64));
  if (grid.y > 65535)
    return fail(kInvalidArgument, "linear fallback has too many rows");
  if (fp8)
    gemm_simt_kernel<true><<<grid, 256, 0, stream>>>(
        args.input, args.weight, ep, static_cast<int>(args.rows),
        static_cast<int>(args.out_features),
        static_cast<int>(args.in_features));
  else
    gemm_simt_kernel<false><<<grid, 256, 0, stream>>>(
        args.input, args.weight, ep, static_cast<int>(args.rows),
        static_cast<int>(args.out_features),
        static_cast<int>(args.in_features));
  return check_launch("CUDA-core GEMM kernel");
}

}  // namespace evob
