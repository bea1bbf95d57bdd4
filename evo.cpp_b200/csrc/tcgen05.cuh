// PTX building blocks shared by the tcgen05 kernels (dense projections,
// attention): mbarriers with time-bounded waits, 2-D TMA tile loads, tcgen05
// MMA / commit / fences, TMEM loads, and the K-major 128-byte-swizzle shared
// memory descriptor.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace evob {
namespace tc {

constexpr unsigned long long kWaitLimitNs = 2000000000ULL;  // 2 s

__device__ __forceinline__ std::uint32_t smem_u32(const void *p) {
  return static_cast<std::uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(const std::uint32_t bar,
                                          const std::uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)
               : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(const std::uint32_t bar,
                                               const std::uint32_t bytes) {
  asm volatile(
      "mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar),
      "r"(bytes)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive(const std::uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded parity wait.  Returns false if the wait was abandoned (either this
// thread ran out of time or another role already raised the abort flag).
__device__ __forceinline__ bool mbar_wait(const std::uint32_t bar,
                                          const std::uint32_t parity,
                                          volatile int *const abort_flag) {
  unsigned long long start = 0;
  for (std::uint32_t spin = 0;; ++spin) {
    std::uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done != 0U) return true;
    if ((spin & 255U) == 255U) {
      if (*abort_flag != 0) return false;
      const unsigned long long now = global_timer_ns();
      if (start == 0) start = now;
      if (now - start > kWaitLimitNs) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}
__device__ __forceinline__ void tma_load_2d(const std::uint32_t dst,
                                            const CUtensorMap *const map,
                                            const std::uint32_t bar,
                                            const int x, const int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::"
      "bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(const std::uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 "
      "[%0];" ::"r"(bar)
      : "memory");
}
template <bool kFp8>
__device__ __forceinline__ void tc_mma(const std::uint32_t tmem_d,
                                       const std::uint64_t desc_a,
                                       const std::uint64_t desc_b,
                                       const std::uint32_t idesc,
                                       const std::uint32_t accumulate) {
  if constexpr (kFp8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(
            tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(
            tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
__device__ __forceinline__ void tmem_load_32(const std::uint32_t taddr,
                                             std::uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, "
      "%30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]),
        "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
        "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
        "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]),
        "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]),
        "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_load_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// K-major, 128-byte swizzle: rows are 128 bytes apart, 8-row groups 1024
// bytes apart; version 1 (Blackwell) descriptor.
__device__ __forceinline__ std::uint64_t smem_descriptor(
    const std::uint32_t address) {
  std::uint64_t desc = 0;
  desc |= static_cast<std::uint64_t>((address & 0x3ffffU) >> 4U);
  desc |= static_cast<std::uint64_t>(1U) << 16U;            // LBO (unused)
  desc |= static_cast<std::uint64_t>(1024U >> 4U) << 32U;   // SBO
  desc |= static_cast<std::uint64_t>(1U) << 46U;            // version
  desc |= static_cast<std::uint64_t>(2U) << 61U;            // SWIZZLE_128B
  return desc;
}


// ---- host side (gemm_tcgen05.cu)
// 2-D BF16 tensor map over a row-major [rows, columns] matrix with boxes of
// 64 columns (one 128-byte swizzle atom) x box_rows rows, SWIZZLE_128B.
int make_bf16_tile_map(CUtensorMap *map, const void *base, std::size_t rows, std::size_t columns,
                       int box_rows);
// Per-device sticky error word raised by a timed-out wait in any tcgen05
// kernel (reported by gemm_error_state); also the device's SM count.
int *error_word(int *status, int *sm_count);

}  // namespace tc
}  // namespace evob
