// Attention for a handful of query rows against a long KV cache (cached
// decode, short continuations): head size 128, same contract as
// causal_attention - row i sees keys 0 .. total_keys - rows + i.
//
// One row and head has almost no parallelism in the query, so the keys are
// split instead: a thread-block cluster of kSplits CTAs shares one (row, head);
// each CTA runs an online softmax over its slice of the keys (8 lanes per key,
// 16 dimensions each, 128-bit loads of K and V), the warps of a CTA merge
// through shared memory, and the CTAs of the cluster merge through distributed
// shared memory - no scratch buffer, one launch.
#include <cooperative_groups.h>

#include "common.cuh"
#include "ops_internal.hpp"

namespace evob {
namespace {
namespace cg = cooperative_groups;

constexpr int kHeadDim = 128;
constexpr int kSplits = 8;          // CTAs per cluster
constexpr int kDecodeThreads = 256;
constexpr int kWarps = kDecodeThreads / 32;
constexpr int kPartial = kHeadDim + 2;  // accumulator, running max, running sum

__device__ __forceinline__ void unpack16(const uint4 a, const uint4 b, float (&out)[16]) {
  const std::uint32_t words[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    out[2 * i] = __uint_as_float(words[i] << 16U);
    out[2 * i + 1] = __uint_as_float(words[i] & 0xffff0000U);
  }
}

// Folds (m, l, acc) of another partial softmax into this one.
__device__ __forceinline__ void merge(float &m, float &l, float &acc, const float other_m,
                                      const float other_l, const float other_acc) {
  const float merged = fmaxf(m, other_m);
  const float mine = m == -INFINITY ? 0.0F : __expf(m - merged);
  const float theirs = other_m == -INFINITY ? 0.0F : __expf(other_m - merged);
  acc = acc * mine + other_acc * theirs;
  l = l * mine + other_l * theirs;
  m = merged;
}

// 16 int8 codes of one 128-bit load times their vector's scale.
__device__ __forceinline__ void unpack16_q8(const uint4 codes, const float scale, float (&out)[16]) {
  const std::uint32_t words[4] = {codes.x, codes.y, codes.z, codes.w};
#pragma unroll
  for (int i = 0; i < 16; ++i)
    out[i] = static_cast<float>(static_cast<std::int8_t>((words[i / 4] >> (8 * (i % 4))) & 0xffU)) * scale;
}

// kQ8: K and V come from the paged int8 cache of the fast-q8-kv profile (`pages`) instead of
// the BF16 caches.
template <bool kQ8>
__global__ void __launch_bounds__(kDecodeThreads)
attention_decode_kernel(const bf16 *__restrict__ query, const bf16 *__restrict__ key_cache,
                        const bf16 *__restrict__ value_cache, const Q8PageTable pages, bf16 *__restrict__ output,
                        const int rows, const int static_total_keys, const int heads,
                        const int *__restrict__ dynamic_prefix) {
  // lets a one-row projection launched with programmatic stream serialisation start (and fetch its
  // weights) under this kernel; it still waits for this grid to finish before it reads the result
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // replayed launches (CUDA graphs) read the number of keys already cached from device memory
  const int total_keys = dynamic_prefix != nullptr ? *dynamic_prefix + rows : static_total_keys;
  __shared__ float warp_partials[kWarps][kPartial];
  __shared__ float cta_partial[kPartial];
  cg::cluster_group cluster = cg::this_cluster();
  const int split = static_cast<int>(cluster.block_rank());
  const int head = blockIdx.y, row = blockIdx.z;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int group = lane / 8, part = lane % 8;  // 4 keys per warp step, 16 dimensions per lane
  const std::size_t width = static_cast<std::size_t>(heads) * kHeadDim;
  const int visible = total_keys - rows + row + 1;
  const int per_split = (visible + kSplits - 1) / kSplits;
  const int key_begin = split * per_split;
  const int key_end = min(visible, key_begin + per_split);
  const float scale = rsqrtf(static_cast<float>(kHeadDim));

  float q[16];
  {
    const uint4 *const source = reinterpret_cast<const uint4 *>(
        query + static_cast<std::size_t>(row) * width + head * kHeadDim + part * 16);
    unpack16(__ldg(source), __ldg(source + 1), q);
  }
  float running_max = -INFINITY, running_sum = 0.0F;
  float acc[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) acc[i] = 0.0F;
  const std::size_t lane_offset = static_cast<std::size_t>(head) * kHeadDim + part * 16;
  for (int key0 = key_begin + warp * 4; key0 < key_end; key0 += kWarps * 4) {
    const int key = key0 + group;
    const bool live = key < key_end;
    float k[16], v[16];
    if (live) {
      if constexpr (kQ8) {
        const std::size_t page = static_cast<std::size_t>(key) / pages.page_tokens;
        const std::size_t slot = (static_cast<std::size_t>(key) % pages.page_tokens) * heads + head;
        const uint4 kc = __ldg(reinterpret_cast<const uint4 *>(pages.key[page] + slot * kHeadDim + part * 16));
        const uint4 vc = __ldg(reinterpret_cast<const uint4 *>(pages.value[page] + slot * kHeadDim + part * 16));
        unpack16_q8(kc, __ldg(pages.key_scale[page] + slot), k);
        unpack16_q8(vc, __ldg(pages.value_scale[page] + slot), v);
      } else {
        const uint4 *const kp = reinterpret_cast<const uint4 *>(key_cache + static_cast<std::size_t>(key) * width + lane_offset);
        const uint4 *const vp = reinterpret_cast<const uint4 *>(value_cache + static_cast<std::size_t>(key) * width + lane_offset);
        const uint4 k0 = __ldg(kp), k1 = __ldg(kp + 1), v0 = __ldg(vp), v1 = __ldg(vp + 1);
        unpack16(k0, k1, k);
        unpack16(v0, v1, v);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) k[i] = v[i] = 0.0F;
    }
    float dot = 0.0F;
#pragma unroll
    for (int i = 0; i < 16; ++i) dot = fmaf(q[i], k[i], dot);
    dot += __shfl_xor_sync(0xffffffffU, dot, 1);
    dot += __shfl_xor_sync(0xffffffffU, dot, 2);
    dot += __shfl_xor_sync(0xffffffffU, dot, 4);
    if (live) {
      const float score = dot * scale;
      const float new_max = fmaxf(running_max, score);
      const float correction = __expf(running_max - new_max);  // exp(-inf) = 0 on the first key
      const float p = __expf(score - new_max);
      running_sum = running_sum * correction + p;
#pragma unroll
      for (int i = 0; i < 16; ++i) acc[i] = fmaf(acc[i], correction, p * v[i]);
      running_max = new_max;
    }
  }
  // the four key groups of a warp hold partials over the same 16 dimensions per `part`
#pragma unroll
  for (int offset = 8; offset <= 16; offset *= 2) {
    const float other_m = __shfl_xor_sync(0xffffffffU, running_max, offset);
    const float other_l = __shfl_xor_sync(0xffffffffU, running_sum, offset);
    const float merged = fmaxf(running_max, other_m);
    const float mine = running_max == -INFINITY ? 0.0F : __expf(running_max - merged);
    const float theirs = other_m == -INFINITY ? 0.0F : __expf(other_m - merged);
#pragma unroll
    for (int i = 0; i < 16; ++i)
      acc[i] = acc[i] * mine + __shfl_xor_sync(0xffffffffU, acc[i], offset) * theirs;
    running_sum = running_sum * mine + other_l * theirs;
    running_max = merged;
  }
  if (group == 0) {
#pragma unroll
    for (int i = 0; i < 16; ++i) warp_partials[warp][part * 16 + i] = acc[i];
    if (part == 0) {
      warp_partials[warp][kHeadDim] = running_max;
      warp_partials[warp][kHeadDim + 1] = running_sum;
    }
  }
  __syncthreads();
  if (threadIdx.x < kHeadDim) {
    float m = warp_partials[0][kHeadDim], l = warp_partials[0][kHeadDim + 1], a = warp_partials[0][threadIdx.x];
    for (int w = 1; w < kWarps; ++w)
      merge(m, l, a, warp_partials[w][kHeadDim], warp_partials[w][kHeadDim + 1], warp_partials[w][threadIdx.x]);
    cta_partial[threadIdx.x] = a;
    if (threadIdx.x == 0) {
      cta_partial[kHeadDim] = m;
      cta_partial[kHeadDim + 1] = l;
    }
  }
  cluster.sync();
  if (split == 0 && threadIdx.x < kHeadDim) {
    float m = cta_partial[kHeadDim], l = cta_partial[kHeadDim + 1], a = cta_partial[threadIdx.x];
    for (int other = 1; other < kSplits; ++other) {
      const float *const remote = cluster.map_shared_rank(cta_partial, other);
      merge(m, l, a, remote[kHeadDim], remote[kHeadDim + 1], remote[threadIdx.x]);
    }
    output[static_cast<std::size_t>(row) * width + head * kHeadDim + threadIdx.x] = f2bf(a / l);
  }
  cluster.sync();  // remote shared memory stays alive until rank 0 has read it
}

}  // namespace

bool attention_decode_applicable(const void *query, const void *key_cache, const void *value_cache,
                                 const std::size_t rows, const std::size_t total_keys, const std::size_t heads,
                                 const std::size_t head_dim, const void *output) {
  if (head_dim != kHeadDim || rows == 0 || rows > 8 || heads == 0 || heads > 65535 || total_keys < rows ||
      total_keys > 0x7fffff00U)
    return false;
  for (const void *p : {query, key_cache, value_cache, output})
    if (p == nullptr || (reinterpret_cast<std::uintptr_t>(p) & 15U) != 0) return false;
  return true;
}

namespace {
template <bool kQ8>
int launch_decode(const void *query, const void *key_cache, const void *value_cache, const Q8PageTable &pages,
                  const std::size_t rows, const std::size_t total_keys, const std::size_t heads, void *output,
                  cudaStream_t stream, const int *dynamic_prefix) {
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(kSplits, static_cast<unsigned int>(heads), static_cast<unsigned int>(rows));
  config.blockDim = dim3(kDecodeThreads);
  config.dynamicSmemBytes = 0;
  config.stream = stream;
  cudaLaunchAttribute attribute{};
  attribute.id = cudaLaunchAttributeClusterDimension;
  attribute.val.clusterDim.x = kSplits;
  attribute.val.clusterDim.y = 1;
  attribute.val.clusterDim.z = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  const cudaError_t error = cudaLaunchKernelEx(
      &config, attention_decode_kernel<kQ8>, static_cast<const bf16 *>(query),
      static_cast<const bf16 *>(key_cache), static_cast<const bf16 *>(value_cache), pages,
      static_cast<bf16 *>(output), static_cast<int>(rows), static_cast<int>(total_keys), static_cast<int>(heads),
      dynamic_prefix);
  if (error != cudaSuccess)
    return fail(kCuda, std::string("attention decode kernel launch failed: ") + cudaGetErrorString(error));
  return check_launch("attention decode kernel");
}
}  // namespace

int attention_decode(const void *query, const void *key_cache, const void *value_cache, const std::size_t rows,
                     const std::size_t total_keys, const std::size_t heads, void *output, cudaStream_t stream,
                     const int *dynamic_prefix) {
  return launch_decode<false>(query, key_cache, value_cache, Q8PageTable{}, rows, total_keys, heads, output, stream,
                              dynamic_prefix);
}

int q8_attention_decode(const void *query, const Q8PageTable &pages, const std::size_t rows,
                        const std::size_t total_keys, const std::size_t heads, const std::size_t head_dim,
                        void *output, cudaStream_t stream) {
  if (query == nullptr || output == nullptr || pages.key == nullptr || pages.value == nullptr ||
      pages.key_scale == nullptr || pages.value_scale == nullptr || pages.page_tokens == 0 || head_dim != kHeadDim ||
      rows == 0 || rows > 8 || heads == 0 || heads > 65535 || total_keys < rows || total_keys > 0x7fffff00U ||
      (reinterpret_cast<std::uintptr_t>(query) & 15U) != 0)
    return fail(kInvalidArgument, "quantised decode attention arguments are invalid (1..8 rows, head size 128)");
  return launch_decode<true>(query, nullptr, nullptr, pages, rows, total_keys, heads, output, stream, nullptr);
}

}  // namespace evob
