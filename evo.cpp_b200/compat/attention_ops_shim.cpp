// evo::cuda attention operators (upstream include/evo/cuda/attention.hpp:13-154) on this library's C
// entry points; see compat_common.hpp for what the layer is.
//
// How the pieces map:
//  * bf16_mha_prefill / bf16_mha_decode: one fused split + RoPE + cache-append kernel, then causal
//    attention over the cache (tcgen05 kernel for 128-wide heads and long chunks, warp-MMA and row-wise
//    kernels otherwise).  The workspace's key / value buffers still receive the rotated keys and the
//    values of the chunk, as upstream leaves them there.
//  * bf16_split_qkv and bf16_kv_append (BF16 cache) are strided device copies; bf16_apply_rope runs the
//    fused kernel on a staged [q | k | 0] image, so its arithmetic is the product's.
//  * The quantised (Q8, paged) cache keeps upstream's layout: pages allocated when first touched,
//    device tables of page pointers, host mirrors.  Chunks attend to a BF16 image rebuilt from the
//    pages; 1..8-row steps at head size 128 read the pages directly.
//  * bf16_cached_cross_attention keeps the scaled keys and the scores on chip; of upstream's three
//    intermediate tensors only the BF16 probabilities are written.  All three scratch buffers are grown
//    to upstream's sizes (and zero-filled when new) so that callers' size assumptions hold.
#include "compat_common.hpp"

#include <algorithm>
#include <utility>

#include "evo/cuda/attention.hpp"

namespace evo::cuda {

using evo_b200_compat::DeviceScope;
using evo_b200_compat::from_code;
using evo_b200_compat::holds;
using evo_b200_compat::invalid;
using evo_b200_compat::kBf16Bytes;
using evo_b200_compat::product;
using evo_b200_compat::StreamScratch;

namespace {

void *raw(const Stream &stream) { return static_cast<void *>(stream.get()); }

bool on_device(const Stream &stream, const DeviceBuffer &buffer) {
  return stream.valid() && buffer.valid() && buffer.device() == stream.device();
}

// Bytes of a BF16 [tokens, heads, head_dim] tensor, or false when a factor is zero or it overflows.
bool tensor_bytes(const std::size_t tokens, const std::size_t heads, const std::size_t head_dim, std::size_t *bytes) {
  std::size_t elements = 0;
  if (tokens == 0 || heads == 0 || head_dim == 0 || !product(tokens, heads, head_dim, &elements)) return false;
  return product(elements, kBf16Bytes, 1, bytes);
}

Status grow(DeviceBuffer *buffer, const int device, const std::size_t bytes) {
  if (buffer == nullptr) return invalid("a scratch buffer pointer is null");
  if (buffer->valid() && buffer->device() == device && buffer->bytes() >= bytes) return Status::Ok();
  return buffer->allocate(device, bytes);
}

// `base` moved back by `rows` rows of `row_bytes`: the fused append kernel addresses its targets by
// absolute position, so a target that starts at position `rows` is handed over as if it started at
// position 0.  The kernel never touches the rows in front.
void *rewound(void *base, const std::size_t rows, const std::size_t row_bytes) {
  return reinterpret_cast<void *>(reinterpret_cast<std::uintptr_t>(base) - rows * row_bytes);
}

struct PageTables final {
  void *const *key;
  void *const *value;
  void *const *key_scale;
  void *const *value_scale;
};

PageTables tables_of(const KvCache &cache) {
  return {static_cast<void *const *>(cache.key_page_table.data()), static_cast<void *const *>(cache.value_page_table.data()),
          static_cast<void *const *>(cache.key_scale_page_table.data()),
          static_cast<void *const *>(cache.value_scale_page_table.data())};
}

Status check_cache(const KvCache &cache, const Stream &stream) {
  if (cache.capacity == 0 || cache.heads == 0 || cache.head_dim == 0 || cache.length > cache.capacity ||
      !stream.valid() || cache.device_id != stream.device())
    return invalid("the KV cache is not allocated on the stream's device");
  if (cache.type == KvCacheType::kBF16) {
    std::size_t bytes = 0;
    if (!tensor_bytes(cache.capacity, cache.heads, cache.head_dim, &bytes) || !holds(cache.key, bytes) ||
        !holds(cache.value, bytes))
      return invalid("the BF16 KV cache buffers do not match its capacity");
    return Status::Ok();
  }
  const std::size_t pages = cache.page_tokens == 0 ? 0 : (cache.capacity + cache.page_tokens - 1) / cache.page_tokens;
  if (pages == 0 || cache.q8_pages.size() != pages || cache.host_key_pages.size() != pages ||
      cache.host_value_pages.size() != pages || cache.host_key_scale_pages.size() != pages ||
      cache.host_value_scale_pages.size() != pages || !holds(cache.key_page_table, pages * sizeof(void *)) ||
      !holds(cache.value_page_table, pages * sizeof(void *)) || !holds(cache.key_scale_page_table, pages * sizeof(void *)) ||
      !holds(cache.value_scale_page_table, pages * sizeof(void *)))
    return invalid("the paged Q8 KV cache tables do not match its capacity");
  return Status::Ok();
}

// Allocates the pages that positions [0, token_end) touch and publishes their addresses in the
// device tables (stream-ordered; the host vectors outlive the copies because the cache does).
Status touch_pages(KvCache *cache, const std::size_t token_end, const Stream &stream) {
  const std::size_t wanted = (token_end + cache->page_tokens - 1) / cache->page_tokens;
  std::size_t code_bytes = 0, scale_bytes = 0;
  if (!product(cache->page_tokens, cache->heads, cache->head_dim, &code_bytes) ||
      !product(cache->page_tokens, cache->heads, sizeof(float), &scale_bytes))
    return invalid("Q8 page size is not representable");
  bool changed = false;
  for (std::size_t page = 0; page < wanted; ++page) {
    Q8KvPage &slot = cache->q8_pages[page];
    if (slot.key.valid()) continue;
    for (DeviceBuffer *const buffer : {&slot.key, &slot.value}) {
      auto status = buffer->allocate(cache->device_id, code_bytes);
      if (!status.ok()) return status;
    }
    for (DeviceBuffer *const buffer : {&slot.key_scale, &slot.value_scale}) {
      auto status = buffer->allocate(cache->device_id, scale_bytes);
      if (!status.ok()) return status;
    }
    cache->host_key_pages[page] = static_cast<std::int8_t *>(slot.key.data());
    cache->host_value_pages[page] = static_cast<std::int8_t *>(slot.value.data());
    cache->host_key_scale_pages[page] = static_cast<float *>(slot.key_scale.data());
    cache->host_value_scale_pages[page] = static_cast<float *>(slot.value_scale.data());
    changed = true;
  }
  if (!changed) return Status::Ok();
  const std::size_t bytes = cache->q8_pages.size() * sizeof(void *);
  auto status = cache->key_page_table.copy_from_host(cache->host_key_pages.data(), bytes, stream);
  if (status.ok()) status = cache->value_page_table.copy_from_host(cache->host_value_pages.data(), bytes, stream);
  if (status.ok()) status = cache->key_scale_page_table.copy_from_host(cache->host_key_scale_pages.data(), bytes, stream);
  if (status.ok())
    status = cache->value_scale_page_table.copy_from_host(cache->host_value_scale_pages.data(), bytes, stream);
  return status;
}

// Causal attention of `rows` queries at positions [prefix, prefix + rows) over the cache.
Status attend(const void *query, const std::size_t rows, const std::size_t prefix, const KvCache &cache, void *output,
              const Stream &stream) {
  const std::size_t total = prefix + rows;
  if (cache.type == KvCacheType::kBF16) {
    return from_code(evo_b200_bf16_causal_attention(query, cache.key.data(), cache.value.data(), rows, total, cache.heads,
                                                    cache.head_dim, output, raw(stream)),
                     "causal attention");
  }
  const PageTables tables = tables_of(cache);
  if (cache.head_dim == 128 && rows <= 8) {
    return from_code(evo_b200_q8_attention_decode(query, tables.key, tables.value, tables.key_scale, tables.value_scale,
                                                  cache.page_tokens, rows, total, cache.heads, cache.head_dim, output,
                                                  raw(stream)),
                     "Q8 cached attention");
  }
  std::size_t bytes = 0;
  if (!tensor_bytes(total, cache.heads, cache.head_dim, &bytes)) return invalid("Q8 attention: the context is too large");
  StreamScratch keys, values;
  auto status = keys.allocate(bytes, stream.get());
  if (status.ok()) status = values.allocate(bytes, stream.get());
  if (!status.ok()) return status;
  status = from_code(evo_b200_q8_kv_expand(tables.key, tables.value, tables.key_scale, tables.value_scale,
                                           cache.page_tokens, total, cache.heads, cache.head_dim, keys.data(),
                                           values.data(), raw(stream)),
                     "Q8 cache expansion");
  if (!status.ok()) return status;
  return from_code(evo_b200_bf16_causal_attention(query, keys.data(), values.data(), rows, total, cache.heads,
                                                  cache.head_dim, output, raw(stream)),
                   "causal attention over the expanded Q8 cache");
}

}  // namespace

// ---- KvCache and AttentionWorkspace -------------------------------------------------------------

Status KvCache::allocate(const int device, const std::size_t token_capacity, const std::size_t head_count,
                         const std::size_t dimensions_per_head) {
  std::size_t bytes = 0;
  if (!tensor_bytes(token_capacity, head_count, dimensions_per_head, &bytes))
    return invalid("KV cache: capacity, heads and head size must be positive and representable");
  auto status = key.allocate(device, bytes);
  if (status.ok()) status = value.allocate(device, bytes);
  if (!status.ok()) return status;
  q8_pages.clear();
  for (DeviceBuffer *const table : {&key_page_table, &value_page_table, &key_scale_page_table, &value_scale_page_table})
    table->reset();
  host_key_pages.clear();
  host_value_pages.clear();
  host_key_scale_pages.clear();
  host_value_scale_pages.clear();
  type = KvCacheType::kBF16;
  device_id = device;
  capacity = token_capacity;
  length = 0;
  heads = head_count;
  head_dim = dimensions_per_head;
  page_tokens = 0;
  return Status::Ok();
}

Status KvCache::allocate_q8_paged(const int device, const std::size_t token_capacity, const std::size_t head_count,
                                  const std::size_t dimensions_per_head, const std::size_t tokens_per_page,
                                  const Stream &stream) {
  std::size_t ignored = 0;
  if (tokens_per_page == 0 || !tensor_bytes(token_capacity, head_count, dimensions_per_head, &ignored) ||
      !tensor_bytes(tokens_per_page, head_count, dimensions_per_head, &ignored))
    return invalid("Q8 KV cache: capacity, heads, head size and page size must be positive and representable");
  if (!stream.valid() || stream.device() != device) return invalid("Q8 KV cache: the stream belongs to another device");
  const std::size_t pages = (token_capacity + tokens_per_page - 1) / tokens_per_page;
  key.reset();
  value.reset();
  q8_pages.clear();
  q8_pages.resize(pages);
  host_key_pages.assign(pages, nullptr);
  host_value_pages.assign(pages, nullptr);
  host_key_scale_pages.assign(pages, nullptr);
  host_value_scale_pages.assign(pages, nullptr);
  for (DeviceBuffer *const table : {&key_page_table, &value_page_table, &key_scale_page_table, &value_scale_page_table}) {
    auto status = table->allocate(device, pages * sizeof(void *));
    if (status.ok()) status = table->zero(stream);
    if (!status.ok()) return status;
  }
  type = KvCacheType::kQ8Paged;
  device_id = device;
  capacity = token_capacity;
  length = 0;
  heads = head_count;
  head_dim = dimensions_per_head;
  page_tokens = tokens_per_page;
  return Status::Ok();
}

std::size_t KvCache::allocated_bytes() const noexcept {
  std::size_t total = key.bytes() + value.bytes() + key_page_table.bytes() + value_page_table.bytes() +
                      key_scale_page_table.bytes() + value_scale_page_table.bytes();
  for (const Q8KvPage &page : q8_pages)
    total += page.key.bytes() + page.value.bytes() + page.key_scale.bytes() + page.value_scale.bytes();
  return total;
}

Status AttentionWorkspace::allocate(const int device, const std::size_t token_count, const std::size_t head_count,
                                    const std::size_t dimensions_per_head) {
  std::size_t bytes = 0, rows = 0;
  if (!tensor_bytes(token_count, head_count, dimensions_per_head, &bytes) ||
      !product(token_count, head_count, sizeof(float), &rows))
    return invalid("attention workspace: tokens, heads and head size must be positive and representable");
  for (DeviceBuffer *const buffer : {&query, &key, &value}) {
    auto status = buffer->allocate(device, bytes);
    if (!status.ok()) return status;
  }
  // one F32 per (token, head): the log-sum-exp slot of upstream's flash kernel; unused by this build's
  // kernels, kept so that code sizing its own scratch from it still finds it
  auto status = softmax_lse.allocate(device, rows);
  if (!status.ok()) return status;
  for (DeviceBuffer *const buffer : {&softmax_lse_accum, &output_accum, &scaled_key, &scores, &probabilities})
    buffer->reset();
  tokens = token_count;
  heads = head_count;
  head_dim = dimensions_per_head;
  return Status::Ok();
}

// ---- the separate steps -------------------------------------------------------------------------

Status bf16_split_qkv(const DeviceBuffer &qkv, const std::size_t tokens, const std::size_t heads,
                      const std::size_t head_dim, DeviceBuffer *const query, DeviceBuffer *const key,
                      DeviceBuffer *const value, const Stream &stream, const QkvLayout layout) {
  std::size_t bytes = 0;
  if (!tensor_bytes(tokens, heads, head_dim, &bytes) || bytes > std::numeric_limits<std::size_t>::max() / 3)
    return invalid("QKV split: tokens, heads and head size must be positive and representable");
  if (!holds(qkv, 3 * bytes) || !holds(query, bytes) || !holds(key, bytes) || !holds(value, bytes) ||
      !on_device(stream, qkv) || !on_device(stream, *query) || !on_device(stream, *key) || !on_device(stream, *value))
    return invalid("QKV split: buffers are missing, too small or on another device");
  // Both layouts are three strided copies: runs of `run` bytes, every 3 * run bytes in the source.
  const std::size_t run = (layout == QkvLayout::kProjectionMajor ? heads * head_dim : head_dim) * kBf16Bytes;
  const std::size_t runs = bytes / run;
  DeviceBuffer *const targets[3] = {query, key, value};
  for (std::size_t part = 0; part < 3; ++part) {
    const auto *const source = static_cast<const unsigned char *>(qkv.data()) + part * run;
    auto status = cuda_status(cudaMemcpy2DAsync(targets[part]->data(), run, source, 3 * run, run, runs,
                                                cudaMemcpyDeviceToDevice, stream.get()),
                              "cudaMemcpy2DAsync (QKV split)");
    if (!status.ok()) return status;
  }
  return Status::Ok();
}

Status bf16_apply_rope(DeviceBuffer *const query, DeviceBuffer *const key, const DeviceBuffer &inverse_frequency,
                       const std::size_t tokens, const std::size_t heads, const std::size_t head_dim,
                       const std::size_t position_offset, const float position_scale, const Stream &stream) {
  std::size_t bytes = 0;
  if (!tensor_bytes(tokens, heads, head_dim, &bytes) || head_dim % 2 != 0 ||
      bytes > std::numeric_limits<std::size_t>::max() / 3)
    return invalid("RoPE: tokens and heads must be positive, the head size even, and the tensor representable");
  if (!(position_scale > 0.0F) || position_scale > std::numeric_limits<float>::max())
    return invalid("RoPE: the position scale must be positive and finite");
  if (position_offset > std::numeric_limits<std::size_t>::max() - tokens) return invalid("RoPE: positions overflow");
  if (!holds(query, bytes) || !holds(key, bytes) || !holds(inverse_frequency, head_dim / 2 * sizeof(float)) ||
      !on_device(stream, *query) || !on_device(stream, *key) || !on_device(stream, inverse_frequency))
    return invalid("RoPE: buffers are missing, too small or on another device");
  // stage [q | k | 0] per token, rotate through the fused kernel back into the callers' buffers
  const std::size_t row = heads * head_dim * kBf16Bytes;
  StreamScratch staged, values;
  auto status = staged.allocate(3 * bytes, stream.get());
  if (status.ok()) status = values.allocate(bytes, stream.get());
  if (!status.ok()) return status;
  status = cuda_status(cudaMemsetAsync(staged.data(), 0, 3 * bytes, stream.get()), "cudaMemsetAsync (RoPE staging)");
  if (!status.ok()) return status;
  DeviceBuffer *const sources[2] = {query, key};
  for (std::size_t part = 0; part < 2; ++part) {
    status = cuda_status(cudaMemcpy2DAsync(static_cast<unsigned char *>(staged.data()) + part * row, 3 * row,
                                           sources[part]->data(), row, row, tokens, cudaMemcpyDeviceToDevice,
                                           stream.get()),
                         "cudaMemcpy2DAsync (RoPE staging)");
    if (!status.ok()) return status;
  }
  return from_code(evo_b200_bf16_split_rope_append(staged.data(), static_cast<const float *>(inverse_frequency.data()),
                                                   tokens, heads, head_dim, position_offset, position_scale, 0,
                                                   query->data(), rewound(key->data(), position_offset, row),
                                                   rewound(values.data(), position_offset, row), position_offset + tokens,
                                                   raw(stream)),
                   "RoPE");
}

Status bf16_kv_append(const DeviceBuffer &key, const DeviceBuffer &value, const std::size_t tokens, KvCache *const cache,
                      const Stream &stream) {
  if (cache == nullptr) return invalid("KV append needs a cache");
  auto status = check_cache(*cache, stream);
  if (!status.ok()) return status;
  std::size_t bytes = 0;
  if (!tensor_bytes(tokens, cache->heads, cache->head_dim, &bytes)) return invalid("KV append: nothing to append");
  if (tokens > cache->capacity - cache->length) return invalid("KV append exceeds the cache capacity");
  if (!holds(key, bytes) || !holds(value, bytes) || !on_device(stream, key) || !on_device(stream, value))
    return invalid("KV append: key or value is missing, too small or on another device");
  if (cache->type == KvCacheType::kBF16) {
    const std::size_t at = cache->length * cache->heads * cache->head_dim * kBf16Bytes;
    status = cuda_status(cudaMemcpyAsync(static_cast<unsigned char *>(cache->key.data()) + at, key.data(), bytes,
                                         cudaMemcpyDeviceToDevice, stream.get()),
                         "cudaMemcpyAsync (key append)");
    if (status.ok())
      status = cuda_status(cudaMemcpyAsync(static_cast<unsigned char *>(cache->value.data()) + at, value.data(), bytes,
                                           cudaMemcpyDeviceToDevice, stream.get()),
                           "cudaMemcpyAsync (value append)");
  } else {
    status = touch_pages(cache, cache->length + tokens, stream);
    if (!status.ok()) return status;
    const PageTables tables = tables_of(*cache);
    status = from_code(evo_b200_q8_kv_append(key.data(), value.data(), tables.key, tables.value, tables.key_scale,
                                             tables.value_scale, cache->page_tokens, cache->length, tokens, cache->heads,
                                             cache->head_dim, raw(stream)),
                       "Q8 KV append");
  }
  if (status.ok()) cache->length += tokens;
  return status;
}

Status bf16_online_causal_attention(const DeviceBuffer &query, const std::size_t query_tokens,
                                    const std::size_t prefix_tokens, const KvCache &cache, DeviceBuffer *const output,
                                    const Stream &stream) {
  auto status = check_cache(cache, stream);
  if (!status.ok()) return status;
  std::size_t bytes = 0;
  if (!tensor_bytes(query_tokens, cache.heads, cache.head_dim, &bytes)) return invalid("causal attention: no queries");
  if (prefix_tokens > cache.length || query_tokens > cache.length - prefix_tokens)
    return invalid("causal attention: the cache holds fewer keys than prefix + queries");
  if (!holds(query, bytes) || !holds(output, bytes) || !on_device(stream, query) || !on_device(stream, *output))
    return invalid("causal attention: query or output is missing, too small or on another device");
  return attend(query.data(), query_tokens, prefix_tokens, cache, output->data(), stream);
}

Status bf16_flash_causal_attention(const DeviceBuffer &query, const DeviceBuffer &key, const DeviceBuffer &value,
                                   const std::size_t query_tokens, const std::size_t key_tokens, const std::size_t heads,
                                   const std::size_t head_dim, DeviceBuffer *const softmax_lse,
                                   DeviceBuffer *const softmax_lse_accum, DeviceBuffer *const output_accum,
                                   DeviceBuffer *const output, const Stream &stream) {
  (void)softmax_lse;        // the kernels of this build keep their softmax statistics on chip and
  (void)softmax_lse_accum;  // never split one row's keys over CTAs in prefill
  (void)output_accum;
  std::size_t query_bytes = 0, key_bytes = 0;
  if (!tensor_bytes(query_tokens, heads, head_dim, &query_bytes) || !tensor_bytes(key_tokens, heads, head_dim, &key_bytes) ||
      key_tokens < query_tokens)
    return invalid("flash attention: sizes must be positive and keys at least as many as queries");
  if (!holds(query, query_bytes) || !holds(key, key_bytes) || !holds(value, key_bytes) || !holds(output, query_bytes) ||
      !on_device(stream, query) || !on_device(stream, key) || !on_device(stream, value) || !on_device(stream, *output))
    return invalid("flash attention: buffers are missing, too small or on another device");
  return from_code(evo_b200_bf16_causal_attention(query.data(), key.data(), value.data(), query_tokens, key_tokens, heads,
                                                  head_dim, output->data(), raw(stream)),
                   "flash attention");
}

Status bf16_cached_cross_attention(const Blas &blas, const DeviceBuffer &query, const DeviceBuffer &key,
                                   const DeviceBuffer &value, const std::size_t query_tokens, const std::size_t key_tokens,
                                   const std::size_t heads, const std::size_t head_dim, DeviceBuffer *const scaled_key,
                                   DeviceBuffer *const scores, DeviceBuffer *const probabilities,
                                   DeviceBuffer *const output, const Stream &stream) {
  if (!blas.valid()) return invalid("cached attention: the BLAS handle has not been created");
  std::size_t query_bytes = 0, key_bytes = 0, score_bytes = 0;
  if (!tensor_bytes(query_tokens, heads, head_dim, &query_bytes) || !tensor_bytes(key_tokens, heads, head_dim, &key_bytes) ||
      !tensor_bytes(query_tokens, heads, key_tokens, &score_bytes) || key_tokens < query_tokens)
    return invalid("cached attention: sizes must be positive and keys at least as many as queries");
  if (!holds(query, query_bytes) || !holds(key, key_bytes) || !holds(value, key_bytes) || !holds(output, query_bytes) ||
      !on_device(stream, query) || !on_device(stream, key) || !on_device(stream, value) || !on_device(stream, *output))
    return invalid("cached attention: buffers are missing, too small or on another device");
  const std::pair<DeviceBuffer *, std::size_t> scratch[3] = {
      {scaled_key, key_bytes}, {scores, score_bytes}, {probabilities, score_bytes}};
  for (const auto &[buffer, bytes] : scratch) {
    const bool fresh = buffer != nullptr && !(buffer->valid() && buffer->bytes() >= bytes);
    auto status = grow(buffer, stream.device(), bytes);
    if (status.ok() && fresh) status = buffer->zero(stream);
    if (!status.ok()) return status;
  }
  return from_code(evo_b200_bf16_cached_cross_attention_probabilities(
                       query.data(), key.data(), value.data(), query_tokens, key_tokens, heads, head_dim,
                       probabilities == nullptr ? nullptr : probabilities->data(), output->data(), raw(stream)),
                   "cached attention");
}

// ---- the whole attention step -------------------------------------------------------------------

Status bf16_mha_prefill(const DeviceBuffer &qkv, const DeviceBuffer &inverse_frequency, const std::size_t tokens,
                        const std::size_t heads, const std::size_t head_dim, const float position_scale,
                        KvCache *const cache, AttentionWorkspace *const workspace, DeviceBuffer *const output,
                        const Stream &stream) {
  if (cache == nullptr || workspace == nullptr || output == nullptr)
    return invalid("MHA: cache, workspace and output are required");
  if (workspace->tokens != tokens || workspace->heads != heads || workspace->head_dim != head_dim ||
      cache->heads != heads || cache->head_dim != head_dim)
    return invalid("MHA: the workspace or the cache was allocated for other dimensions");
  auto status = check_cache(*cache, stream);
  if (!status.ok()) return status;
  std::size_t bytes = 0;
  if (!tensor_bytes(tokens, heads, head_dim, &bytes) || head_dim % 2 != 0 ||
      bytes > std::numeric_limits<std::size_t>::max() / 3)
    return invalid("MHA: tokens and heads must be positive and the head size even");
  if (tokens > cache->capacity - cache->length) return invalid("MHA: the chunk does not fit the KV cache");
  if (!holds(qkv, 3 * bytes) || !holds(inverse_frequency, head_dim / 2 * sizeof(float)) || !holds(output, bytes) ||
      !holds(workspace->query, bytes) || !holds(workspace->key, bytes) || !holds(workspace->value, bytes) ||
      !on_device(stream, qkv) || !on_device(stream, inverse_frequency) || !on_device(stream, *output) ||
      !on_device(stream, workspace->query))
    return invalid("MHA: buffers are missing, too small or on another device");

  const std::size_t prefix = cache->length;
  const std::size_t row = heads * head_dim * kBf16Bytes;
  const auto *const frequency = static_cast<const float *>(inverse_frequency.data());
  if (cache->type == KvCacheType::kBF16) {
    status = from_code(evo_b200_bf16_split_rope_append(qkv.data(), frequency, tokens, heads, head_dim, prefix,
                                                       position_scale, 0, workspace->query.data(), cache->key.data(),
                                                       cache->value.data(), cache->capacity, raw(stream)),
                       "MHA split, RoPE and append");
    if (!status.ok()) return status;
    // the chunk's rotated keys and its values, where upstream's separate steps leave them
    status = cuda_status(cudaMemcpyAsync(workspace->key.data(), static_cast<unsigned char *>(cache->key.data()) + prefix * row,
                                         bytes, cudaMemcpyDeviceToDevice, stream.get()),
                         "cudaMemcpyAsync (workspace keys)");
    if (status.ok())
      status = cuda_status(cudaMemcpyAsync(workspace->value.data(),
                                           static_cast<unsigned char *>(cache->value.data()) + prefix * row, bytes,
                                           cudaMemcpyDeviceToDevice, stream.get()),
                           "cudaMemcpyAsync (workspace values)");
    if (!status.ok()) return status;
  } else {
    status = from_code(evo_b200_bf16_split_rope_append(qkv.data(), frequency, tokens, heads, head_dim, prefix,
                                                       position_scale, 0, workspace->query.data(),
                                                       rewound(workspace->key.data(), prefix, row),
                                                       rewound(workspace->value.data(), prefix, row), prefix + tokens,
                                                       raw(stream)),
                       "MHA split and RoPE");
    if (!status.ok()) return status;
    status = touch_pages(cache, prefix + tokens, stream);
    if (!status.ok()) return status;
    const PageTables tables = tables_of(*cache);
    status = from_code(evo_b200_q8_kv_append(workspace->key.data(), workspace->value.data(), tables.key, tables.value,
                                             tables.key_scale, tables.value_scale, cache->page_tokens, prefix, tokens, heads,
                                             head_dim, raw(stream)),
                       "MHA Q8 append");
    if (!status.ok()) return status;
  }
  cache->length = prefix + tokens;
  status = attend(workspace->query.data(), tokens, prefix, *cache, output->data(), stream);
  if (!status.ok()) cache->length = prefix;
  return status;
}

Status bf16_mha_decode(const DeviceBuffer &qkv, const DeviceBuffer &inverse_frequency, const std::size_t heads,
                       const std::size_t head_dim, const float position_scale, KvCache *const cache,
                       AttentionWorkspace *const workspace, DeviceBuffer *const output, const Stream &stream) {
  if (workspace == nullptr || workspace->tokens != 1) return invalid("MHA decode needs a workspace allocated for one token");
  return bf16_mha_prefill(qkv, inverse_frequency, 1, heads, head_dim, position_scale, cache, workspace, output, stream);
}

}  // namespace evo::cuda
