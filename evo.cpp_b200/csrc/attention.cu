// Attention stripe helpers: fused QKV split + RoPE + KV-cache append, and a
// row-wise attention kernel (one CTA per query row and head) that serves
// cached decode, cached ("exact") prefill with upstream's BF16 score and
// probability materialisation, and prefill for head sizes the tensor-core
// kernel does not take.
//
// Numerics follow src/cuda/attention.cu:210-339 (split, NeoX half-pair RoPE
// with BF16-rounded sin/cos, K*scale in BF16, BF16 scores, F32 softmax, BF16
// probabilities) and src/cuda/attention.cu:879-968 (F32 online path).
#include "common.cuh"
#include "ops_internal.hpp"

namespace evob {
namespace {

__global__ void split_rope_append_kernel(
    const bf16 *__restrict__ qkv, const float *__restrict__ inverse_frequency,
    bf16 *__restrict__ query, bf16 *__restrict__ key_cache,
    bf16 *__restrict__ value_cache, const std::size_t rows,
    const std::size_t heads, const std::size_t head_dim,
    const std::size_t position_offset, const float position_scale,
    const bool head_major) {
  const std::size_t half = head_dim / 2;
  const std::size_t width = heads * head_dim;
  const std::size_t elements = rows * heads * half;
  const std::size_t stride = static_cast<std::size_t>(blockDim.x) * gridDim.x;
  for (std::size_t i = static_cast<std::size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
       i < elements; i += stride) {
    const std::size_t pair = i % half;
    const std::size_t head = (i / half) % heads;
    const std::size_t token = i / (half * heads);
    const bf16 *const source = qkv + token * width * 3;
    std::size_t q_at, k_at, v_at;
    if (head_major) {
      q_at = head * 3 * head_dim;
      k_at = q_at + head_dim;
      v_at = k_at + head_dim;
    } else {
      q_at = head * head_dim;
      k_at = width + q_at;
      v_at = 2 * width + q_at;
    }
    const float position =
        static_cast<float>(position_offset + token) / position_scale;
    float sine, cosine;
    sincosf(position * inverse_frequency[pair], &sine, &cosine);
    sine = rbf(sine);
    cosine = rbf(cosine);
    const std::size_t out = token * width + head * head_dim;
    const std::size_t cache = (position_offset + token) * width + head * head_dim;
    const float q1 = bf2f(source[q_at + pair]);
    const float q2 = bf2f(source[q_at + half + pair]);
    query[out + pair] = f2bf(q1 * cosine - q2 * sine);
    query[out + half + pair] = f2bf(q2 * cosine + q1 * sine);
    const float k1 = bf2f(source[k_at + pair]);
    const float k2 = bf2f(source[k_at + half + pair]);
    key_cache[cache + pair] = f2bf(k1 * cosine - k2 * sine);
    key_cache[cache + half + pair] = f2bf(k2 * cosine + k1 * sine);
    value_cache[cache + pair] = source[v_at + pair];
    value_cache[cache + half + pair] = source[v_at + half + pair];
  }
}

// Vectorised form: a thread owns 8 rotation pairs (two 16-byte runs) of
// kHeads consecutive heads of one token, so the sines and cosines - which do
// not depend on the head - are computed once per kHeads heads and every
// access is a 128-bit one.  Same expressions as the scalar kernel above.
template <int kHeads>
__global__ void __launch_bounds__(256)
split_rope_append_vec_kernel(const bf16 *__restrict__ qkv, const float *__restrict__ inverse_frequency,
                             bf16 *__restrict__ query, bf16 *__restrict__ key_cache,
                             bf16 *__restrict__ value_cache, const std::size_t rows,
                             const std::size_t heads, const std::size_t head_dim,
                             const std::size_t static_position_offset, const float position_scale,
                             const bool head_major, const int *__restrict__ dynamic_position) {
  // replayed launches (CUDA graphs) read the position from device memory
  const std::size_t position_offset =
      dynamic_position != nullptr ? static_cast<std::size_t>(*dynamic_position) : static_position_offset;
  const std::size_t half = head_dim / 2;
  const std::size_t width = heads * head_dim;
  const std::size_t groups = half / 8;
  const std::size_t head_blocks = heads / kHeads;
  const std::size_t total = rows * head_blocks * groups;
  const std::size_t stride = static_cast<std::size_t>(blockDim.x) * gridDim.x;
  for (std::size_t i = static_cast<std::size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += stride) {
    const std::size_t pair = (i % groups) * 8;
    const std::size_t head_block = (i / groups) % head_blocks;
    const std::size_t token = i / (groups * head_blocks);
    const float position = static_cast<float>(position_offset + token) / position_scale;
    float sine[8], cosine[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      sincosf(position * inverse_frequency[pair + j], &sine[j], &cosine[j]);
      sine[j] = rbf(sine[j]);
      cosine[j] = rbf(cosine[j]);
    }
    const bf16 *const source = qkv + token * width * 3;
    const auto rotate = [&](const Bf16x8 &low, const Bf16x8 &high, bf16 *const out) {
      uint4 first, second;
      unsigned int *const f = &first.x, *const g = &second.x;
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        const float a0 = low.get(j), b0 = high.get(j), a1 = low.get(j + 1), b1 = high.get(j + 1);
        f[j / 2] = pack_bf16x2(a0 * cosine[j] - b0 * sine[j], a1 * cosine[j + 1] - b1 * sine[j + 1]);
        g[j / 2] = pack_bf16x2(b0 * cosine[j] + a0 * sine[j], b1 * cosine[j + 1] + a1 * sine[j + 1]);
      }
      *reinterpret_cast<uint4 *>(out + pair) = first;
      *reinterpret_cast<uint4 *>(out + half + pair) = second;
    };
#pragma unroll
    for (int h = 0; h < kHeads; ++h) {
      const std::size_t head = head_block * kHeads + h;
      std::size_t q_at, k_at, v_at;
      if (head_major) {
        q_at = head * 3 * head_dim;
        k_at = q_at + head_dim;
        v_at = k_at + head_dim;
      } else {
        q_at = head * head_dim;
        k_at = width + q_at;
        v_at = 2 * width + q_at;
      }
      Bf16x8 q_low, q_high, k_low, k_high;
      q_low.raw = *reinterpret_cast<const uint4 *>(source + q_at + pair);
      q_high.raw = *reinterpret_cast<const uint4 *>(source + q_at + half + pair);
      k_low.raw = *reinterpret_cast<const uint4 *>(source + k_at + pair);
      k_high.raw = *reinterpret_cast<const uint4 *>(source + k_at + half + pair);
      const uint4 v_low = *reinterpret_cast<const uint4 *>(source + v_at + pair);
      const uint4 v_high = *reinterpret_cast<const uint4 *>(source + v_at + half + pair);
      const std::size_t cache = (position_offset + token) * width + head * head_dim;
      rotate(q_low, q_high, query + token * width + head * head_dim);
      rotate(k_low, k_high, key_cache + cache);
      *reinterpret_cast<uint4 *>(value_cache + cache + pair) = v_low;
      *reinterpret_cast<uint4 *>(value_cache + cache + half + pair) = v_high;
    }
  }
}

constexpr int kRowThreads = 128;

__device__ __forceinline__ float block_reduce(float value, float *scratch,
                                              const bool take_max) {
#pragma unroll
  for (int offset = 16; offset > 0; offset /= 2) {
    const float other = __shfl_xor_sync(0xffffffffU, value, offset);
    value = take_max ? fmaxf(value, other) : value + other;
  }
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  __syncthreads();
  if (lane == 0) scratch[warp] = value;
  __syncthreads();
  float result = scratch[0];
  for (int w = 1; w < kRowThreads / 32; ++w)
    result = take_max ? fmaxf(result, scratch[w]) : result + scratch[w];
  return result;
}

// grid (rows, heads); dynamic shared memory: head_dim + visible keys floats.
template <bool kCachedRounding>
__global__ void __launch_bounds__(kRowThreads)
attention_row_kernel(const bf16 *__restrict__ query,
                     const bf16 *__restrict__ key_cache,
                     const bf16 *__restrict__ value_cache,
                     bf16 *__restrict__ output, const int rows,
                     const int total_keys, const int heads,
                     const int head_dim, bf16 *__restrict__ probabilities) {
  extern __shared__ float shared[];
  __shared__ float reduce_scratch[kRowThreads / 32];
  float *const q = shared;
  float *const scores = shared + head_dim;
  const int row = blockIdx.x, head = blockIdx.y;
  const std::size_t width = static_cast<std::size_t>(heads) * head_dim;
  const int visible = total_keys - rows + row + 1;
  const float scale = rsqrtf(static_cast<float>(head_dim));
  for (int d = threadIdx.x; d < head_dim; d += kRowThreads)
    q[d] = bf2f(query[static_cast<std::size_t>(row) * width + head * head_dim + d]);
  __syncthreads();
  float local_max = -INFINITY;
  for (int j = threadIdx.x; j < visible; j += kRowThreads) {
    const bf16 *const k = key_cache + static_cast<std::size_t>(j) * width + head * head_dim;
    float dot = 0.0F;
    for (int d = 0; d < head_dim; ++d) {
      const float kv = kCachedRounding ? rbf(bf2f(k[d]) * scale) : bf2f(k[d]);
      dot = fmaf(q[d], kv, dot);
    }
    const float s = kCachedRounding ? rbf(dot) : dot * scale;
    scores[j] = s;
    local_max = fmaxf(local_max, s);
  }
  const float row_max = block_reduce(local_max, reduce_scratch, true);
  float local_sum = 0.0F;
  for (int j = threadIdx.x; j < visible; j += kRowThreads) {
    const float e = expf(scores[j] - row_max);
    scores[j] = e;
    local_sum += e;
  }
  const float row_sum = block_reduce(local_sum, reduce_scratch, false);
  __syncthreads();
  if (kCachedRounding && probabilities != nullptr) {
    // [heads, rows, total_keys] BF16, zeros behind the causal boundary: the tensor upstream's cached
    // path materialises between its two GEMMs
    bf16 *const target = probabilities + (static_cast<std::size_t>(head) * rows + row) * total_keys;
    for (int j = threadIdx.x; j < total_keys; j += kRowThreads)
      target[j] = f2bf(j < visible ? scores[j] / row_sum : 0.0F);
  }
  // probabilities x values.  The block's threads form `lanes` key lanes x `dims` output dimensions;
  // a thread walks every lanes-th key with four running sums (keys 0, 4, 8, ... of its own sequence in
  // the first, and so on), the lanes' partial sums are then added in lane order.  One running sum over
  // ten thousand keys loses enough low bits to move a BF16 result (it did at 10,240 keys against the
  // reference bytes of upstream's known-answer test); blocked sums do not, and they overlap the loads.
  __shared__ float lane_sums[kRowThreads];
  const int dims = min(head_dim, kRowThreads);
  const int lanes = kRowThreads / dims;
  const int lane = threadIdx.x / dims;
  for (int d0 = 0; d0 < head_dim; d0 += dims) {
    const int d = d0 + threadIdx.x % dims;
    const bool active = lane < lanes && d < head_dim;
    float sums[4] = {0.0F, 0.0F, 0.0F, 0.0F};
    if (active) {
      const bf16 *const v = value_cache + head * head_dim + d;
      int turn = 0;
      for (int j = lane; j < visible; j += lanes, turn = (turn + 1) & 3) {
        const float p = kCachedRounding ? rbf(scores[j] / row_sum) : scores[j];
        sums[turn] = fmaf(p, bf2f(v[static_cast<std::size_t>(j) * width]), sums[turn]);
      }
    }
    __syncthreads();  // the previous pass has read lane_sums
    lane_sums[threadIdx.x] = (sums[0] + sums[1]) + (sums[2] + sums[3]);
    __syncthreads();
    if (active && lane == 0) {
      float acc = lane_sums[threadIdx.x];
      for (int other = 1; other < lanes; ++other) acc += lane_sums[other * dims + threadIdx.x];
      if (!kCachedRounding) acc /= row_sum;
      output[static_cast<std::size_t>(row) * width + head * head_dim + d] = f2bf(acc);
    }
  }
}

template <bool kCachedRounding>
int launch_rows(const void *query, const void *key_cache,
                const void *value_cache, const std::size_t rows,
                const std::size_t total_keys, const std::size_t heads,
                const std::size_t head_dim, void *output, cudaStream_t stream, void *probabilities = nullptr) {
  if (query == nullptr || key_cache == nullptr || value_cache == nullptr ||
      output == nullptr || heads == 0 || head_dim == 0 || total_keys < rows ||
      heads > 65535 || total_keys > 0x7fffffffU)
    return fail(kInvalidArgument, "attention arguments are invalid");
  if (rows == 0) return kOk;
  const std::size_t smem = (head_dim + total_keys) * sizeof(float);
  if (smem > 200 * 1024)
    return fail(kUnsupported,
                "row-wise attention supports at most ~51k visible keys");
  auto *const kernel = attention_row_kernel<kCachedRounding>;
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(smem)) != cudaSuccess)
    return fail(kCuda, "cannot raise the attention shared-memory limit");
  kernel<<<dim3(static_cast<unsigned int>(rows), static_cast<unsigned int>(heads)),
           kRowThreads, smem, stream>>>(
      static_cast<const bf16 *>(query), static_cast<const bf16 *>(key_cache),
      static_cast<const bf16 *>(value_cache), static_cast<bf16 *>(output),
      static_cast<int>(rows), static_cast<int>(total_keys),
      static_cast<int>(heads), static_cast<int>(head_dim), static_cast<bf16 *>(probabilities));
  return check_launch("row-wise attention kernel");
}

}  // namespace

int split_rope_append(const void *qkv, const float *inverse_frequency,
                      const std::size_t rows, const std::size_t heads,
                      const std::size_t head_dim,
                      const std::size_t position_offset,
                      const float position_scale, const bool head_major,
                      void *query, void *key_cache, void *value_cache,
                      const std::size_t cache_capacity, cudaStream_t stream,
                      const int *dynamic_position) {
  if (qkv == nullptr || inverse_frequency == nullptr || query == nullptr ||
      key_cache == nullptr || value_cache == nullptr || heads == 0 ||
      head_dim == 0 || head_dim % 2 != 0 || !(position_scale > 0.0F))
    return fail(kInvalidArgument, "QKV split arguments are invalid");
  if (position_offset + rows > cache_capacity)
    return fail(kInvalidArgument, "KV cache capacity exceeded");
  if (rows == 0) return kOk;
  const std::size_t cap = static_cast<std::size_t>(kSmCount) * 16;
  const auto aligned = [](const void *p) { return reinterpret_cast<std::uintptr_t>(p) % 16 == 0; };
  if (head_dim % 16 == 0 && aligned(qkv) && aligned(query) && aligned(key_cache) && aligned(value_cache)) {
    const bool four = heads % 4 == 0;
    const std::size_t threads = rows * (heads / (four ? 4 : 1)) * (head_dim / 16);
    const std::size_t wanted = (threads + 255) / 256;
    const unsigned int grid = static_cast<unsigned int>(wanted > cap ? cap : wanted);
    const auto kernel = four ? split_rope_append_vec_kernel<4> : split_rope_append_vec_kernel<1>;
    kernel<<<grid, 256, 0, stream>>>(static_cast<const bf16 *>(qkv), inverse_frequency,
                                     static_cast<bf16 *>(query), static_cast<bf16 *>(key_cache),
                                     static_cast<bf16 *>(value_cache), rows, heads, head_dim,
                                     position_offset, position_scale, head_major, dynamic_position);
    return check_launch("QKV split/RoPE/append kernel");
  }
  if (dynamic_position != nullptr)
    return fail(kUnsupported, "a device-side position needs the vectorised split kernel");
  const std::size_t elements = rows * heads * (head_dim / 2);
  const std::size_t blocks = (elements + 255) / 256;
  split_rope_append_kernel<<<static_cast<unsigned int>(blocks > cap ? cap : blocks),
                             256, 0, stream>>>(
      static_cast<const bf16 *>(qkv), inverse_frequency,
      static_cast<bf16 *>(query), static_cast<bf16 *>(key_cache),
      static_cast<bf16 *>(value_cache), rows, heads, head_dim, position_offset,
      position_scale, head_major);
  return check_launch("QKV split/RoPE/append kernel");
}

int flash_causal_attention(const void *query, const void *key_cache,
                           const void *value_cache, std::size_t rows,
                           std::size_t total_keys, std::size_t heads,
                           void *output, cudaStream_t stream);

bool flash_tcgen05_applicable(const void *query, const void *key_cache, const void *value_cache,
                              std::size_t rows, std::size_t total_keys, std::size_t heads,
                              const void *output);
int flash_tcgen05_attention(const void *query, const void *key_cache, const void *value_cache,
                            std::size_t rows, std::size_t total_keys, std::size_t heads,
                            void *output, cudaStream_t stream);

int causal_attention_mma_sync(const void *query, const void *key_cache,
                              const void *value_cache, const std::size_t rows,
                              const std::size_t total_keys, const std::size_t heads,
                              const std::size_t head_dim, void *output,
                              cudaStream_t stream) {
  if (head_dim == 128 && rows >= 16)
    return flash_causal_attention(query, key_cache, value_cache, rows,
                                  total_keys, heads, output, stream);
  return launch_rows<false>(query, key_cache, value_cache, rows, total_keys,
                            heads, head_dim, output, stream);
}

bool attention_decode_applicable(const void *query, const void *key_cache, const void *value_cache,
                                 std::size_t rows, std::size_t total_keys, std::size_t heads,
                                 std::size_t head_dim, const void *output);
int attention_decode(const void *query, const void *key_cache, const void *value_cache, std::size_t rows,
                     std::size_t total_keys, std::size_t heads, void *output, cudaStream_t stream,
                     const int *dynamic_prefix);

int causal_attention(const void *query, const void *key_cache,
                     const void *value_cache, const std::size_t rows,
                     const std::size_t total_keys, const std::size_t heads,
                     const std::size_t head_dim, void *output,
                     cudaStream_t stream, const int *dynamic_prefix) {
  if (attention_decode_applicable(query, key_cache, value_cache, rows, total_keys, heads, head_dim, output))
    return attention_decode(query, key_cache, value_cache, rows, total_keys, heads, output, stream,
                            dynamic_prefix);
  if (dynamic_prefix != nullptr)
    return fail(kUnsupported, "a device-side prefix needs the split-KV attention kernel");
  if (head_dim == 128 && query != nullptr && key_cache != nullptr && value_cache != nullptr &&
      output != nullptr &&
      flash_tcgen05_applicable(query, key_cache, value_cache, rows, total_keys, heads, output))
    return flash_tcgen05_attention(query, key_cache, value_cache, rows, total_keys, heads, output,
                                   stream);
  if (head_dim == 128 && rows >= 16)
    return flash_causal_attention(query, key_cache, value_cache, rows,
                                  total_keys, heads, output, stream);
  return launch_rows<false>(query, key_cache, value_cache, rows, total_keys,
                            heads, head_dim, output, stream);
}

int cached_attention(const void *query, const void *key_cache,
                     const void *value_cache, const std::size_t rows,
                     const std::size_t total_keys, const std::size_t heads,
                     const std::size_t head_dim, void *output,
                     cudaStream_t stream, void *probabilities) {
  return launch_rows<true>(query, key_cache, value_cache, rows, total_keys,
                           heads, head_dim, output, stream, probabilities);
}

}  // namespace evob
