// Small-batch projections (1..8 rows: cached decode and very short prompts).
// At these sizes a projection is a weight stream: every weight byte is read
// once and the arithmetic is negligible, so the tensor-core tile kernel (which
// launches one CTA per 128 x 256 tile and leaves most SMs idle) is replaced by
// a kernel in which a CTA owns a few weight rows, its threads split K in
// 16-byte chunks, and partial sums are folded with shuffles and shared memory.  Same epilogue
// contract as the tile kernel (scale, fused or separately rounded bias,
// residual, gate over row-interleaved up-projections).
#include <cuda_fp8.h>

#include "common.cuh"
#include "ops_internal.hpp"

namespace evob {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxRows = 8;

struct GemvParams {
  const void *x;       // [rows, K] BF16 or E4M3 codes
  const void *w;       // [N, K] same type
  const bf16 *bias, *residual;
  bf16 *out;
  int rows, K, N;      // N = weight rows
  float alpha;
  int bias_mode, gate_mode;
  int dependent_launch;  // launched with programmatic stream serialisation: see the kernel
};

template <bool kFp8>
__device__ __forceinline__ void unpack16(const uint4 raw, float (&v)[kFp8 ? 16 : 8]) {
  if constexpr (kFp8) {
    const unsigned int words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const __half2_raw pair = __nv_cvt_fp8x2_to_halfraw2(
            static_cast<__nv_fp8x2_storage_t>((words[i] >> (16 * h)) & 0xffffU), __NV_E4M3);
        const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&pair));
        v[4 * i + 2 * h] = f.x;
        v[4 * i + 2 * h + 1] = f.y;
      }
    }
  } else {
    Bf16x8 packed;
    packed.raw = raw;
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = packed.get(i);
  }
}

__device__ __forceinline__ bf16 gelu_round_small(const float x) {
  const bf16 input = f2bf(x);
  const float value = bf2f(input);
  const bf16 computed = f2bf(value * 0.5F * (1.0F + ::erff(value * 0.70710678118654752440F)));
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

// A CTA owns kColumns weight rows and its eight warps split K between them, so
// the whole weight slab of the CTA (kColumns x K) is requested within the first
// couple of loop iterations - at one row a projection is a latency problem as
// much as a bandwidth one.  Per-warp partial sums are folded with shuffles,
// then across warps through shared memory; the last step applies the same
// epilogue as the tile kernel.  kRows is a compile-time bound on the rows held
// in registers.
constexpr int kWarps = kThreads / 32;

template <bool kFp8, int kRows, int kColumns>
__global__ void __launch_bounds__(kThreads)
gemv_kernel(const GemvParams p) {
  constexpr int kPerChunk = kFp8 ? 16 : 8;   // elements per 16-byte chunk
  __shared__ float partial[kWarps][kColumns][kRows];
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const bool gated = p.gate_mode != 0;
  // Output columns handled by this CTA.  When gated, the weight holds blocks
  // of 128 first-projection rows followed by the matching 128 second-projection
  // rows; an output column needs one row of each.
  const int out_columns = gated ? p.N / 2 : p.N;
  const int per_cta = gated ? kColumns / 2 : kColumns;
  const int column0 = blockIdx.x * per_cta;
  int weight_row[kColumns];
#pragma unroll
  for (int c = 0; c < kColumns; ++c) {
    const int column = min(column0 + (gated ? c / 2 : c), out_columns - 1);
    weight_row[c] = gated ? (column / 128) * 256 + column % 128 + (c % 2) * 128 : column;
  }
  float acc[kColumns][kRows];
#pragma unroll
  for (int c = 0; c < kColumns; ++c)
#pragma unroll
    for (int r = 0; r < kRows; ++r) acc[c][r] = 0.0F;
  const int chunks = p.K / kPerChunk;
  const std::size_t row_bytes = static_cast<std::size_t>(p.K) * (kFp8 ? 1 : 2);
  const unsigned char *const wb = static_cast<const unsigned char *>(p.w);
  const unsigned char *const xb = static_cast<const unsigned char *>(p.x);
  // Programmatic dependent launch (one-row steps inside the captured decode graph): this grid may be
  // started while the kernel that produces x is still running.  The weights do not depend on that
  // kernel, so the CTA first asks L2 for its weight rows, lets the grid after it start as well, and only
  // then waits for the producer to finish and its writes to be visible.  Without such a launch the two
  // instructions do nothing.
  if (p.dependent_launch != 0) {
    for (int chunk = threadIdx.x * 8; chunk < chunks; chunk += kThreads * 8) {  // one request per 128-byte line
#pragma unroll
      for (int c = 0; c < kColumns; ++c)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(wb + weight_row[c] * row_bytes + static_cast<std::size_t>(chunk) * 16));
    }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
  }
#pragma unroll(kRows == 1 ? 4 : (kRows == 2 ? 2 : 1))
  for (int chunk = threadIdx.x; chunk < chunks; chunk += kThreads) {
    uint4 wraw[kColumns];
#pragma unroll
    for (int c = 0; c < kColumns; ++c)
      wraw[c] = __ldcs(reinterpret_cast<const uint4 *>(wb + weight_row[c] * row_bytes) + chunk);
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      if (r < p.rows) {
        float xv[kPerChunk];
        unpack16<kFp8>(__ldg(reinterpret_cast<const uint4 *>(xb + r * row_bytes) + chunk), xv);
#pragma unroll
        for (int c = 0; c < kColumns; ++c) {
          float wv[kPerChunk];
          unpack16<kFp8>(wraw[c], wv);
#pragma unroll
          for (int i = 0; i < kPerChunk; ++i) acc[c][r] = fmaf(xv[i], wv[i], acc[c][r]);
        }
      }
    }
  }
#pragma unroll
  for (int c = 0; c < kColumns; ++c)
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
#pragma unroll
      for (int offset = 16; offset > 0; offset /= 2)
        acc[c][r] += __shfl_xor_sync(0xffffffffU, acc[c][r], offset);
      if (lane == 0) partial[warp][c][r] = acc[c][r];
    }
  __syncthreads();
  // one thread per (row, output column of the CTA)
  const int item = threadIdx.x;
  if (item >= per_cta * kRows) return;
  const int r = item / per_cta, local = item % per_cta;
  const int column = column0 + local;
  if (r >= p.rows || column >= out_columns) return;
  const auto total = [&](const int c) {
    float sum = 0.0F;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) sum += partial[w][c][r];
    return sum;
  };
  bf16 *const out_row = p.out + static_cast<std::size_t>(r) * out_columns;
  if (gated) {
    const float first = total(2 * local) * p.alpha, second = rbf(total(2 * local + 1) * p.alpha);
    const float activated = p.gate_mode == 2 ? bf2f(gelu_round_small(first)) : rbf(first);
    out_row[column] = f2bf(activated * second);
  } else {
    float value = total(local) * p.alpha;
    if (p.bias_mode == 1) value += bf2f(p.bias[column]);
    value = rbf(value);
    if (p.bias_mode == 2) value = rbf(value + bf2f(p.bias[column]));
    if (p.residual != nullptr)
      value = rbf(value + bf2f(p.residual[static_cast<std::size_t>(r) * out_columns + column]));
    out_row[column] = f2bf(value);
  }
}

// Four weight rows per CTA measured best at every width of the 7B and 40B
// shapes (one row, BF16: 2.7 TB/s at 4096 x 4096, 5.3 TB/s at 22528 x 4096, with four
// 16-byte loads per weight row in flight per thread);
// a gated projection then produces two output columns per CTA.
constexpr int kColumnsPerCta = 4;

template <bool kFp8>
int launch_gemv(const GemvParams &p, cudaStream_t stream) {
  const int out_columns = p.gate_mode != 0 ? p.N / 2 : p.N;
  const int per_cta = p.gate_mode != 0 ? kColumnsPerCta / 2 : kColumnsPerCta;
  const unsigned int grid = static_cast<unsigned int>((out_columns + per_cta - 1) / per_cta);
  if (p.rows == 1 && p.dependent_launch != 0) {
    cudaLaunchAttribute attribute{};
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t config{};
    config.gridDim = dim3(grid);
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = 0;
    config.stream = stream;
    config.attrs = &attribute;
    config.numAttrs = 1;
    if (cudaLaunchKernelEx(&config, gemv_kernel<kFp8, 1, kColumnsPerCta>, p) != cudaSuccess)
      return fail(kCuda, "cannot launch the small-batch projection kernel");
  } else if (p.rows == 1)
    gemv_kernel<kFp8, 1, kColumnsPerCta><<<grid, kThreads, 0, stream>>>(p);
  else if (p.rows <= 2)
    gemv_kernel<kFp8, 2, kColumnsPerCta><<<grid, kThreads, 0, stream>>>(p);
  else if (p.rows <= 4)
    gemv_kernel<kFp8, 4, kColumnsPerCta><<<grid, kThreads, 0, stream>>>(p);
  else
    gemv_kernel<kFp8, 8, kColumnsPerCta><<<grid, kThreads, 0, stream>>>(p);
  return check_launch("small-batch projection kernel");
}

}  // namespace

bool small_batch_linear_applicable(const LinearArgs &a) {
  const bool fp8 = a.operand_type == OperandType::kE4m3;
  const std::size_t per_chunk = fp8 ? 16 : 8;
  return a.rows >= 1 && a.rows <= static_cast<std::size_t>(kMaxRows) && !a.force_simt &&
         a.in_features % per_chunk == 0 && a.in_features >= per_chunk &&
         (reinterpret_cast<std::uintptr_t>(a.input) & 15U) == 0 &&
         (reinterpret_cast<std::uintptr_t>(a.weight) & 15U) == 0 &&
         a.out_features <= 0x7fffffffU && a.in_features <= 0x7fffffffU &&
         (a.gate_mode == 0 || a.out_features % 256 == 0);
}

int small_batch_linear(const LinearArgs &a, cudaStream_t stream) {
  GemvParams p{};
  p.x = a.input;
  p.w = a.weight;
  p.bias = static_cast<const bf16 *>(a.bias);
  p.residual = static_cast<const bf16 *>(a.residual);
  p.out = static_cast<bf16 *>(a.output);
  p.rows = static_cast<int>(a.rows);
  p.K = static_cast<int>(a.in_features);
  p.N = static_cast<int>(a.out_features);
  p.alpha = a.alpha;
  p.bias_mode = a.bias_mode;
  p.gate_mode = a.gate_mode;
  p.dependent_launch = a.dependent_launch && a.rows == 1 ? 1 : 0;
  return a.operand_type == OperandType::kE4m3 ? launch_gemv<true>(p, stream)
                                              : launch_gemv<false>(p, stream);
}

}  // namespace evob
