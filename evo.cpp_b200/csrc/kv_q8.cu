// Quantised KV cache of the fast-q8-kv execution profile (upstream
// docs/execution-profiles.md:96-127; src/cuda/attention.cu:798-866, 1072-1141):
// K and V live in fixed pages of 16,384 tokens as int8, every (token, head)
// vector with its own F32 scale = max|v| / 127 (1 for a zero vector) and
// q = clamp(rint(v / scale), -127, 127); attention sees q * scale.
//
// Upstream quantises with one block per (token, head) and attends with one
// block per (query row, head) walking all keys serially.  Here a warp owns a
// (token, head) vector (four dimensions per lane, 64-bit loads, a shuffle
// maximum, one 32-bit store of four codes); prefill chunks attend through the
// tensor-core kernels on a BF16 image of the visible keys rebuilt from the pages
// (so the values it sees are the quantised ones, as upstream's are), and decode
// steps read the pages directly in the cluster split-KV kernel
// (attention_decode.cu), 16 codes per 128-bit load.
#include <algorithm>

#include "common.cuh"
#include "ops_internal.hpp"

namespace evob {
namespace {

constexpr int kThreads = 256;
constexpr int kHeadDim = 128;

__device__ __forceinline__ float warp_max_all(float value) {
#pragma unroll
  for (int offset = 16; offset > 0; offset /= 2) value = fmaxf(value, __shfl_xor_sync(0xffffffffU, value, offset));
  return value;
}

// rows x heads vectors of the BF16 [rows, heads, 128] tensor -> codes and scales of
// positions first_position .. first_position + rows - 1.
__global__ void __launch_bounds__(kThreads)
q8_append_kernel(const bf16 *__restrict__ key, const bf16 *__restrict__ value, const Q8PageTable pages,
                 const std::size_t first_position, const std::size_t rows, const int heads) {
  const std::size_t vector = (static_cast<std::size_t>(blockIdx.x) * kThreads + threadIdx.x) / 32;
  const int lane = threadIdx.x % 32;
  if (vector >= rows * heads) return;
  const std::size_t row = vector / heads;
  const int head = static_cast<int>(vector % heads);
  const std::size_t position = first_position + row;
  const std::size_t page = position / pages.page_tokens, within = position % pages.page_tokens;
  const std::size_t slot = within * heads + head;  // vector index inside the page
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    const bf16 *const source = (which == 0 ? key : value) + vector * kHeadDim + lane * 4;
    const uint2 raw = *reinterpret_cast<const uint2 *>(source);
    const float x[4] = {__uint_as_float(raw.x << 16U), __uint_as_float(raw.x & 0xffff0000U),
                        __uint_as_float(raw.y << 16U), __uint_as_float(raw.y & 0xffff0000U)};
    const float largest =
        warp_max_all(fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3]))));
    const float scale = largest == 0.0F ? 1.0F : __fdiv_rn(largest, 127.0F);
    std::uint32_t packed = 0U;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int q = max(-127, min(127, __float2int_rn(__fdiv_rn(x[i], scale))));
      packed |= static_cast<std::uint32_t>(static_cast<std::uint8_t>(static_cast<std::int8_t>(q))) << (8 * i);
    }
    std::int8_t *const codes = (which == 0 ? pages.key : pages.value)[page];
    *reinterpret_cast<std::uint32_t *>(codes + slot * kHeadDim + lane * 4) = packed;
    if (lane == 0) (which == 0 ? pages.key_scale : pages.value_scale)[page][slot] = scale;
  }
}

// positions [0, count) of the pages -> BF16 [count, heads, 128] images of K and V.
__global__ void __launch_bounds__(kThreads)
q8_expand_kernel(const Q8PageTable pages, bf16 *__restrict__ key, bf16 *__restrict__ value, const std::size_t count,
                 const int heads) {
  const std::size_t vector = (static_cast<std::size_t>(blockIdx.x) * kThreads + threadIdx.x) / 32;
  const int lane = threadIdx.x % 32;
  if (vector >= count * heads) return;
  const std::size_t position = vector / heads;
  const int head = static_cast<int>(vector % heads);
  const std::size_t page = position / pages.page_tokens, within = position % pages.page_tokens;
  const std::size_t slot = within * heads + head;
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    const std::int8_t *const codes = (which == 0 ? pages.key : pages.value)[page];
    const float scale = (which == 0 ? pages.key_scale : pages.value_scale)[page][slot];
    const std::uint32_t packed = *reinterpret_cast<const std::uint32_t *>(codes + slot * kHeadDim + lane * 4);
    float x[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
      x[i] = static_cast<float>(static_cast<std::int8_t>((packed >> (8 * i)) & 0xffU)) * scale;
    bf16 *const target = (which == 0 ? key : value) + vector * kHeadDim + lane * 4;
    *reinterpret_cast<uint2 *>(target) = make_uint2(pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]));
  }
}

// The same two operators for any head size (the model shapes all use 128): a warp still owns a
// (token, head) vector, its lanes stride over the dimensions one element at a time.
__global__ void __launch_bounds__(kThreads)
q8_append_any_kernel(const bf16 *__restrict__ key, const bf16 *__restrict__ value, const Q8PageTable pages,
                     const std::size_t first_position, const std::size_t rows, const int heads, const int head_dim) {
  const std::size_t vector = (static_cast<std::size_t>(blockIdx.x) * kThreads + threadIdx.x) / 32;
  const int lane = threadIdx.x % 32;
  if (vector >= rows * heads) return;
  const std::size_t position = first_position + vector / heads;
  const int head = static_cast<int>(vector % heads);
  const std::size_t page = position / pages.page_tokens, within = position % pages.page_tokens;
  const std::size_t slot = within * heads + head;
  for (int which = 0; which < 2; ++which) {
    const bf16 *const source = (which == 0 ? key : value) + vector * head_dim;
    float largest = 0.0F;
    for (int d = lane; d < head_dim; d += 32) largest = fmaxf(largest, fabsf(bf2f(source[d])));
    largest = warp_max_all(largest);
    const float scale = largest == 0.0F ? 1.0F : __fdiv_rn(largest, 127.0F);
    std::int8_t *const codes = (which == 0 ? pages.key : pages.value)[page] + slot * head_dim;
    for (int d = lane; d < head_dim; d += 32)
      codes[d] = static_cast<std::int8_t>(max(-127, min(127, __float2int_rn(__fdiv_rn(bf2f(source[d]), scale)))));
    if (lane == 0) (which == 0 ? pages.key_scale : pages.value_scale)[page][slot] = scale;
  }
}

__global__ void __launch_bounds__(kThreads)
q8_expand_any_kernel(const Q8PageTable pages, bf16 *__restrict__ key, bf16 *__restrict__ value, const std::size_t count,
                     const int heads, const int head_dim) {
  const std::size_t vector = (static_cast<std::size_t>(blockIdx.x) * kThreads + threadIdx.x) / 32;
  const int lane = threadIdx.x % 32;
  if (vector >= count * heads) return;
  const std::size_t position = vector / heads;
  const int head = static_cast<int>(vector % heads);
  const std::size_t page = position / pages.page_tokens, within = position % pages.page_tokens;
  const std::size_t slot = within * heads + head;
  for (int which = 0; which < 2; ++which) {
    const std::int8_t *const codes = (which == 0 ? pages.key : pages.value)[page] + slot * head_dim;
    const float scale = (which == 0 ? pages.key_scale : pages.value_scale)[page][slot];
    bf16 *const target = (which == 0 ? key : value) + vector * head_dim;
    for (int d = lane; d < head_dim; d += 32) target[d] = f2bf(static_cast<float>(codes[d]) * scale);
  }
}

int check_table(const Q8PageTable &pages, const std::size_t heads, const std::size_t head_dim) {
  if (pages.key == nullptr || pages.value == nullptr || pages.key_scale == nullptr || pages.value_scale == nullptr ||
      pages.page_tokens == 0 || heads == 0 || heads > 0x7fffU || head_dim == 0 || head_dim > 0x7fffU)
    return fail(kInvalidArgument, "quantised KV cache arguments are invalid");
  return kOk;
}

}  // namespace

int q8_kv_append(const void *key, const void *value, const Q8PageTable &pages, const std::size_t first_position,
                 const std::size_t rows, const std::size_t heads, const std::size_t head_dim, cudaStream_t stream) {
  const int status = check_table(pages, heads, head_dim);
  if (status != kOk) return status;
  if (key == nullptr || value == nullptr) return fail(kInvalidArgument, "quantised KV append needs K and V");
  if (rows == 0) return kOk;
  const std::size_t warps = rows * heads;
  if (warps > 0x3ffffffU) return fail(kInvalidArgument, "quantised KV append is too large");
  if (head_dim != kHeadDim) {
    q8_append_any_kernel<<<ceil_div_u(warps * 32, kThreads), kThreads, 0, stream>>>(
        static_cast<const bf16 *>(key), static_cast<const bf16 *>(value), pages, first_position, rows,
        static_cast<int>(heads), static_cast<int>(head_dim));
    return check_launch("quantised KV append kernel");
  }
  if ((reinterpret_cast<std::uintptr_t>(key) & 7U) != 0 || (reinterpret_cast<std::uintptr_t>(value) & 7U) != 0)
    return fail(kInvalidArgument, "quantised KV append needs 8-byte aligned K and V");
  q8_append_kernel<<<ceil_div_u(warps * 32, kThreads), kThreads, 0, stream>>>(
      static_cast<const bf16 *>(key), static_cast<const bf16 *>(value), pages, first_position, rows,
      static_cast<int>(heads));
  return check_launch("quantised KV append kernel");
}

int q8_kv_expand(const Q8PageTable &pages, const std::size_t count, const std::size_t heads,
                 const std::size_t head_dim, void *key, void *value, cudaStream_t stream) {
  const int status = check_table(pages, heads, head_dim);
  if (status != kOk) return status;
  if (key == nullptr || value == nullptr) return fail(kInvalidArgument, "quantised KV expansion needs outputs");
  if (head_dim == kHeadDim &&
      ((reinterpret_cast<std::uintptr_t>(key) & 7U) != 0 || (reinterpret_cast<std::uintptr_t>(value) & 7U) != 0))
    return fail(kInvalidArgument, "quantised KV expansion needs 8-byte aligned outputs");
  if (count == 0) return kOk;
  const std::size_t warps = count * heads;
  if (warps > 0x3ffffffU) {
    // long contexts: one launch per 2^25 vectors
    const std::size_t step = std::max<std::size_t>(1, (std::size_t{1} << 25) / heads / pages.page_tokens) * pages.page_tokens;
    for (std::size_t begin = 0; begin < count; begin += step) {
      Q8PageTable shifted = pages;
      if (begin % pages.page_tokens != 0) return fail(kInternal, "quantised KV expansion step must align to pages");
      shifted.key += begin / pages.page_tokens;
      shifted.value += begin / pages.page_tokens;
      shifted.key_scale += begin / pages.page_tokens;
      shifted.value_scale += begin / pages.page_tokens;
      const std::size_t part = std::min(step, count - begin);
      const int inner = q8_kv_expand(shifted, part, heads, head_dim,
                                     static_cast<bf16 *>(key) + begin * heads * head_dim,
                                     static_cast<bf16 *>(value) + begin * heads * head_dim, stream);
      if (inner != kOk) return inner;
    }
    return kOk;
  }
  if (head_dim != kHeadDim) {
    q8_expand_any_kernel<<<ceil_div_u(warps * 32, kThreads), kThreads, 0, stream>>>(
        pages, static_cast<bf16 *>(key), static_cast<bf16 *>(value), count, static_cast<int>(heads),
        static_cast<int>(head_dim));
    return check_launch("quantised KV expansion kernel");
  }
  q8_expand_kernel<<<ceil_div_u(warps * 32, kThreads), kThreads, 0, stream>>>(
      pages, static_cast<bf16 *>(key), static_cast<bf16 *>(value), count, static_cast<int>(heads));
  return check_launch("quantised KV expansion kernel");
}

}  // namespace evob
