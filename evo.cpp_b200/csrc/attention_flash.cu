// Causal prefill attention for head size 128: a FlashAttention-2 style
// single-pass kernel (online softmax in the exp2 domain, F32 accumulators,
// BF16 probabilities for the P.V product) on warp-level m16n8k16 BF16 MMAs.
// One 4-warp CTA owns 64 query rows of one head and streams 64-key K/V tiles
// through a double-buffered, XOR-swizzled shared-memory ring filled with
// cp.async.  Same mathematical contract as upstream's FlashAttention-2 call
// (src/cuda/flash_attention.cu:199-441): softmax(Q K^T / sqrt(128)) V with
// query i seeing keys 0 .. prefix + i.
#include "common.cuh"
#include "ops_internal.hpp"

namespace evob {
namespace {

constexpr int kHeadDim = 128;
constexpr int kBlockM = 64;
constexpr int kBlockN = 64;
constexpr int kFlashThreads = 128;
constexpr int kRowBytes = kHeadDim * 2;  // 256
constexpr int kTileBytes = kBlockN * kRowBytes;

__device__ __forceinline__ std::uint32_t swizzled(const int row, const int chunk) {
  return static_cast<std::uint32_t>(row * kRowBytes + ((chunk ^ (row & 7)) << 4));
}
__device__ __forceinline__ void cp_async_16(const std::uint32_t dst, const void *src,
                                            const bool valid) {
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
  asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int kPending>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(const std::uint32_t address,
                                            std::uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(address));
}
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

// Copies up to 64 rows x 256 bytes of one head into a swizzled tile.
__device__ __forceinline__ void load_tile(const std::uint32_t tile,
                                          const bf16 *base, const int first_row,
                                          const int row_limit,
                                          const std::size_t row_stride) {
#pragma unroll
  for (int i = 0; i < (kBlockN * 16) / kFlashThreads; ++i) {
    const int item = threadIdx.x + i * kFlashThreads;
    const int row = item / 16, chunk = item % 16;
    const int global_row = first_row + row;
    const bool valid = global_row < row_limit;
    const bf16 *const src =
        base + static_cast<std::size_t>(valid ? global_row : 0) * row_stride + chunk * 8;
    cp_async_16(tile + swizzled(row, chunk), src, valid);
  }
}

__global__ void __launch_bounds__(kFlashThreads)
flash_causal_kernel(const bf16 *__restrict__ query, const bf16 *__restrict__ key_cache,
                    const bf16 *__restrict__ value_cache, bf16 *__restrict__ output,
                    const int rows, const int total_keys, const int heads) {
  extern __shared__ __align__(128) unsigned char flash_smem[];
  const std::uint32_t q_tile = static_cast<std::uint32_t>(__cvta_generic_to_shared(flash_smem));
  const std::uint32_t k_tiles = q_tile + kTileBytes;
  const std::uint32_t v_tiles = k_tiles + 2 * kTileBytes;

  const int block = gridDim.x - 1 - blockIdx.x;  // heaviest (latest) rows first
  const int head = blockIdx.y;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int m0 = block * kBlockM;
  const int prefix = total_keys - rows;
  const std::size_t stride = static_cast<std::size_t>(heads) * kHeadDim;
  const bf16 *const q_base = query + head * kHeadDim;
  const bf16 *const k_base = key_cache + head * kHeadDim;
  const bf16 *const v_base = value_cache + head * kHeadDim;

  const int last_key = min(total_keys, prefix + m0 + kBlockM);  // exclusive
  const int key_blocks = (last_key + kBlockN - 1) / kBlockN;

  load_tile(q_tile, q_base, m0, rows, stride);
  load_tile(k_tiles, k_base, 0, total_keys, stride);
  load_tile(v_tiles, v_base, 0, total_keys, stride);
  cp_async_commit();

  const float scale_log2 = 1.4426950408889634F * rsqrtf(static_cast<float>(kHeadDim));
  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o[i][j] = 0.0F;
  std::uint32_t q_frag[kHeadDim / 16][4];
  float row_max[2] = {-INFINITY, -INFINITY};
  float row_sum[2] = {0.0F, 0.0F};
  const int q_row0 = m0 + warp * 16 + lane / 4;  // and +8

  for (int kb = 0; kb < key_blocks; ++kb) {
    const int buffer = kb & 1;
    if (kb + 1 < key_blocks) {
      load_tile(k_tiles + (buffer ^ 1) * kTileBytes, k_base, (kb + 1) * kBlockN,
                total_keys, stride);
      load_tile(v_tiles + (buffer ^ 1) * kTileBytes, v_base, (kb + 1) * kBlockN,
                total_keys, stride);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const std::uint32_t k_tile = k_tiles + buffer * kTileBytes;
    const std::uint32_t v_tile = v_tiles + buffer * kTileBytes;

    // ---- S = Q K^T (16 x 64 per warp)
    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = 0.0F;
    if (kb == 0) {
      // Q fragments stay in registers for the whole key loop.
#pragma unroll
      for (int ks = 0; ks < kHeadDim / 16; ++ks)
        ldmatrix_x4(q_tile + swizzled(warp * 16 + (lane % 16), 2 * ks + lane / 16), q_frag[ks]);
    }
#pragma unroll
    for (int ks = 0; ks < kHeadDim / 16; ++ks) {
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        std::uint32_t b[4];
        ldmatrix_x4(k_tile + swizzled(16 * np + (lane % 8) + (lane / 16) * 8,
                                      2 * ks + ((lane / 8) % 2)),
                    b);
        mma_bf16(s[2 * np], q_frag[ks], b[0], b[1]);
        mma_bf16(s[2 * np + 1], q_frag[ks], b[2], b[3]);
      }
    }

    // ---- mask + online softmax
    const int key0 = kb * kBlockN + (lane % 4) * 2;
    const bool needs_mask = (kb + 1) * kBlockN > prefix + m0 + 1 ||
                            (kb + 1) * kBlockN > total_keys;
    float block_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int half = j / 2;
        float value = s[nt][j] * scale_log2;
        if (needs_mask) {
          const int key = key0 + nt * 8 + (j & 1);
          const int q_row = q_row0 + half * 8;
          if (key > prefix + q_row || key >= total_keys) value = -INFINITY;
        }
        s[nt][j] = value;
        block_max[half] = fmaxf(block_max[half], value);
      }
    float correction[2];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      float m = block_max[half];
      m = fmaxf(m, __shfl_xor_sync(0xffffffffU, m, 1));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffU, m, 2));
      const float updated = fmaxf(row_max[half], m);
      const float safe = updated == -INFINITY ? 0.0F : updated;
      correction[half] = exp2f(row_max[half] - safe);
      row_max[half] = updated;
      block_max[half] = safe;
      row_sum[half] *= correction[half];
    }
    std::uint32_t p[4][4];  // A fragments of P for the 4 key k-steps
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const float p0 = exp2f(s[nt][0] - block_max[0]);
      const float p1 = exp2f(s[nt][1] - block_max[0]);
      const float p2 = exp2f(s[nt][2] - block_max[1]);
      const float p3 = exp2f(s[nt][3] - block_max[1]);
      row_sum[0] += p0 + p1;
      row_sum[1] += p2 + p3;
      p[nt / 2][(nt % 2) * 2] = pack_bf16x2(p0, p1);
      p[nt / 2][(nt % 2) * 2 + 1] = pack_bf16x2(p2, p3);
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      o[i][0] *= correction[0];
      o[i][1] *= correction[0];
      o[i][2] *= correction[1];
      o[i][3] *= correction[1];
    }

    // ---- O += P V
#pragma unroll
    for (int kk = 0; kk < kBlockN / 16; ++kk) {
#pragma unroll
      for (int dp = 0; dp < kHeadDim / 16; ++dp) {
        std::uint32_t b[4];
        ldmatrix_x4_trans(v_tile + swizzled(16 * kk + (lane % 8) + ((lane / 8) % 2) * 8,
                                            2 * dp + lane / 16),
                          b);
        mma_bf16(o[2 * dp], p[kk], b[0], b[1]);
        mma_bf16(o[2 * dp + 1], p[kk], b[2], b[3]);
      }
    }
    __syncthreads();
  }

#pragma unroll
  for (int half = 0; half < 2; ++half) {
    float total = row_sum[half];
    total += __shfl_xor_sync(0xffffffffU, total, 1);
    total += __shfl_xor_sync(0xffffffffU, total, 2);
    row_sum[half] = total > 0.0F ? 1.0F / total : 0.0F;
  }
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int q_row = q_row0 + half * 8;
    if (q_row >= rows) continue;
    bf16 *const out = output + static_cast<std::size_t>(q_row) * stride + head * kHeadDim +
                      (lane % 4) * 2;
#pragma unroll
    for (int nt = 0; nt < 16; ++nt)
      *reinterpret_cast<std::uint32_t *>(out + nt * 8) =
          pack_bf16x2(o[nt][half * 2] * row_sum[half], o[nt][half * 2 + 1] * row_sum[half]);
  }
}

}  // namespace

int flash_causal_attention(const void *query, const void *key_cache,
                           const void *value_cache, const std::size_t rows,
                           const std::size_t total_keys, const std::size_t heads,
                           void *output, cudaStream_t stream) {
  if (query == nullptr || key_cache == nullptr || value_cache == nullptr ||
      output == nullptr || heads == 0 || heads > 65535 || total_keys < rows ||
      total_keys > 0x7fffff00U)
    return fail(kInvalidArgument, "flash attention arguments are invalid");
  if (rows == 0) return kOk;
  for (const void *p : {query, key_cache, value_cache, static_cast<const void *>(output)})
    if ((reinterpret_cast<std::uintptr_t>(p) & 15U) != 0)
      return fail(kInvalidArgument, "flash attention buffers must be 16-byte aligned");
  constexpr int smem = 5 * kTileBytes;
  // per device and cheap: set on every call
  if (cudaFuncSetAttribute(flash_causal_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           smem) != cudaSuccess)
    return fail(kCuda, "cannot raise the flash attention shared-memory limit");
  const dim3 grid(ceil_div_u(rows, kBlockM), static_cast<unsigned int>(heads));
  flash_causal_kernel<<<grid, kFlashThreads, smem, stream>>>(
      static_cast<const bf16 *>(query), static_cast<const bf16 *>(key_cache),
      static_cast<const bf16 *>(value_cache), static_cast<bf16 *>(output),
      static_cast<int>(rows), static_cast<int>(total_keys), static_cast<int>(heads));
  return check_launch("flash attention kernel");
}

}  // namespace evob
