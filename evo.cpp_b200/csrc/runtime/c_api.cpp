// The evo_* C ABI (include/evo/evo.h) over the sm_100a runtime.  Behaviour
// follows upstream src/c_api.cpp: opaque handles, null-safe frees, parameter
// structs validated through struct_size, thread-local error text, exceptions
// never cross the boundary, a context is poisoned by any failure after its
// state may have advanced (src/c_api.cpp:862-1073).
#include "../../../include/evo/evo.h"
#include "../../../include/evo/evo_b200.h"

#include <algorithm>
#include <cstring>
#include <exception>
#include <functional>
#include <memory>
#include <new>
#include <string>
#include <vector>

#include "../common.cuh"
#include "../ops_internal.hpp"
#include "model.hpp"
#include "sampler.hpp"
#include "scheduler.hpp"
#include "variant.hpp"
#include "variant_io.hpp"

struct evo_model {
  std::shared_ptr<evob::ModelFile> file;
  std::shared_ptr<evob::ModelWeights> weights;
};
struct evo_context {
  std::unique_ptr<evob::Context> context;
  bool failed = false;
  std::string profile;
};
struct evo_batch {
  std::size_t capacity = 0;
  std::vector<std::vector<std::uint8_t>> sequences;
};
struct evo_b200_scheduler {
  std::unique_ptr<evob::Scheduler> scheduler;
};
struct evo_b200_reference {
  std::unique_ptr<evob::ReferenceFasta> fasta;
};
struct evo_sampler {
  explicit evo_sampler(const evob::SamplingConfig &config) : sampler(config) {}
  evob::Sampler sampler;
};

namespace {

using evob::fail;
using evob::kOk;

template <typename F>
evo_status protect(F &&body) {
  try {
    const int status = body();
    if (status == kOk) evob::set_error(kOk, "");
    return static_cast<evo_status>(status);
  } catch (const std::bad_alloc &) {
    return static_cast<evo_status>(fail(evob::kInternal, "out of host memory"));
  } catch (const std::exception &error) {
    return static_cast<evo_status>(fail(evob::kInternal, error.what()));
  } catch (...) {
    return static_cast<evo_status>(fail(evob::kInternal, "unknown exception"));
  }
}

bool valid_status(const evo_status status) {
  switch (status) {
    case EVO_STATUS_OK: case EVO_STATUS_INVALID_ARGUMENT: case EVO_STATUS_IO:
    case EVO_STATUS_MODEL_FORMAT: case EVO_STATUS_UNSUPPORTED: case EVO_STATUS_CUDA:
    case EVO_STATUS_MPS: case EVO_STATUS_INTERNAL: return true;
  }
  return false;
}

int single_sequence_tokens(const evo_batch *batch, std::vector<std::uint32_t> *tokens) {
  if (batch->sequences.size() != 1)
    return fail(evob::kInvalidArgument, "a batch must hold exactly one sequence (batch size 1)");
  const auto &sequence = batch->sequences.front();
  if (sequence.empty()) return fail(evob::kInvalidArgument, "sequence is empty");
  tokens->assign(sequence.begin(), sequence.end());  // identity byte tokenizer
  return kOk;
}

}  // namespace

extern "C" {

uint32_t evo_abi_version(void) { return EVO_ABI_VERSION_CURRENT; }
const char *evo_version_string(void) { return "0.1.0+b200"; }

const char *evo_status_name(const evo_status status) {
  switch (status) {
    case EVO_STATUS_OK: return "ok";
    case EVO_STATUS_INVALID_ARGUMENT: return "invalid_argument";
    case EVO_STATUS_IO: return "io";
    case EVO_STATUS_MODEL_FORMAT: return "model_format";
    case EVO_STATUS_UNSUPPORTED: return "unsupported";
    case EVO_STATUS_CUDA: return "cuda";
    case EVO_STATUS_MPS: return "mps";
    case EVO_STATUS_INTERNAL: return "internal";
  }
  return "unknown";
}

const char *evo_backend_name(const evo_backend backend) {
  switch (backend) {
    case EVO_BACKEND_AUTO: return "auto";
    case EVO_BACKEND_CUDA: return "cuda";
    case EVO_BACKEND_CPU: return "cpu";
    case EVO_BACKEND_MPS: return "mps";
  }
  return "unknown";
}

const char *evo_last_error(void) { return evob::last_error(); }

evo_model_params evo_model_default_params(void) {
  evo_model_params p{};
  p.struct_size = sizeof(p);
  p.backend = EVO_BACKEND_AUTO;
  return p;
}
evo_context_params evo_context_default_params(void) {
  evo_context_params p{};
  p.struct_size = sizeof(p);
  p.context_size = 4096;
  return p;
}
evo_sampler_params evo_sampler_default_params(void) {
  evo_sampler_params p{};
  p.struct_size = sizeof(p);
  p.temperature = 1.0F;
  p.top_k = 1;
  p.top_p = 1.0F;
  p.seed = 0;
  return p;
}
evo_embedding_options evo_embedding_default_options(void) {
  evo_embedding_options o{};
  o.struct_size = sizeof(o);
  o.layer = static_cast<size_t>(-1);
  return o;
}

evo_status evo_model_load(const char *path, const evo_model_params *params, evo_model **model_out) {
  return protect([&]() -> int {
    if (model_out != nullptr) *model_out = nullptr;
    if (path == nullptr || model_out == nullptr)
      return fail(evob::kInvalidArgument, "model path and output are required");
    evo_model_params p = evo_model_default_params();
    if (params != nullptr) {
      if (params->struct_size < sizeof(evo_model_params))
        return fail(evob::kInvalidArgument, "evo_model_params.struct_size is too small");
      p = *params;
    }
    if (p.backend != EVO_BACKEND_AUTO && p.backend != EVO_BACKEND_CUDA)
      return fail(evob::kUnsupported, "this library provides the CUDA backend only");
    if (p.device_count != 0 && p.devices == nullptr)
      return fail(evob::kInvalidArgument, "device list is null");
    std::vector<int> devices(p.devices, p.devices + p.device_count);
    if (devices.empty()) devices.push_back(0);
    auto model = std::make_unique<evo_model>();
    int status = evob::ModelFile::open(path, &model->file);
    if (status != kOk) return status;
    status = evob::load_weights(*model->file, devices,
                                (p.flags & EVO_MODEL_FLAG_TEST_ONLY_ALLOW_SYNTHETIC) != 0, 0,
                                &model->weights);
    if (status != kOk) return status;
    *model_out = model.release();
    return kOk;
  });
}

void evo_model_free(evo_model *model) { delete model; }
evo_backend evo_model_backend(const evo_model *model) {
  return model == nullptr ? EVO_BACKEND_AUTO : EVO_BACKEND_CUDA;
}
const char *evo_model_id(const evo_model *model) {
  return model == nullptr ? "" : model->weights->config.model_id.c_str();
}
const char *evo_model_architecture(const evo_model *model) {
  return model == nullptr ? "" : model->weights->config.architecture.c_str();
}
const char *evo_model_profile(const evo_model *model) {
  return model == nullptr ? "" : model->weights->config.artifact_profile.c_str();
}
size_t evo_model_vocab_size(const evo_model *model) {
  return model == nullptr ? 0 : model->weights->config.vocab;
}
size_t evo_model_max_context(const evo_model *model) {
  return model == nullptr ? 0 : model->weights->config.max_seqlen;
}
size_t evo_model_embedding_width(const evo_model *model) {
  return model == nullptr ? 0 : model->weights->config.width;
}
size_t evo_model_layer_count(const evo_model *model) {
  return model == nullptr ? 0 : model->weights->config.layers;
}

evo_status evo_model_encode(const evo_model *model, const uint8_t *sequence, size_t length,
                            uint32_t *tokens, size_t capacity, size_t *count) {
  return protect([&]() -> int {
    if (model == nullptr || count == nullptr || (sequence == nullptr && length != 0))
      return fail(evob::kInvalidArgument, "encode arguments are invalid");
    *count = length;
    if (tokens == nullptr) return kOk;
    if (capacity < length) return fail(evob::kInvalidArgument, "token buffer is too small");
    for (size_t i = 0; i < length; ++i) tokens[i] = sequence[i];
    return kOk;
  });
}

evo_status evo_model_decode_token(const evo_model *model, uint32_t token, uint8_t *byte_out) {
  return protect([&]() -> int {
    if (model == nullptr || byte_out == nullptr)
      return fail(evob::kInvalidArgument, "decode arguments are invalid");
    if (token > 255) return fail(evob::kInvalidArgument, "token does not map to a byte");
    *byte_out = static_cast<uint8_t>(token);
    return kOk;
  });
}

evo_status evo_context_create(const evo_model *model, const evo_context_params *params,
                              evo_context **context_out) {
  return protect([&]() -> int {
    if (context_out != nullptr) *context_out = nullptr;
    if (model == nullptr || context_out == nullptr)
      return fail(evob::kInvalidArgument, "model and context output are required");
    evo_context_params p = evo_context_default_params();
    if (params != nullptr) {
      if (params->struct_size < sizeof(evo_context_params))
        return fail(evob::kInvalidArgument, "evo_context_params.struct_size is too small");
      p = *params;
    }
    const bool q8_kv = (p.flags & EVO_CONTEXT_FLAG_FAST_Q8_KV) != 0;
    const bool fp8_ffn = (p.flags & EVO_CONTEXT_FLAG_B200_FP8_FFN) != 0;
    const bool tensor_core = fp8_ffn || (p.flags & EVO_CONTEXT_FLAG_B200_TENSORCORE_FP8) != 0;
    auto context = std::make_unique<evo_context>();
    context->profile = fp8_ffn ? "b200-fp8" : tensor_core ? "b200-tc" : "exact";
    // upstream's name for the quantised-cache profile; the projection profile is appended when
    // it is not the default
    if (q8_kv) context->profile = context->profile == "exact" ? "fast-q8-kv" : "fast-q8-kv+" + context->profile;
    const int status = evob::Context::create(
        model->weights, p.context_size,
        fp8_ffn       ? evob::ExecutionProfile::kTensorCoreFfn
        : tensor_core ? evob::ExecutionProfile::kTensorCore
                      : evob::ExecutionProfile::kExact,
        (p.flags & EVO_CONTEXT_FLAG_B200_FULL_ARENA) != 0, &context->context, q8_kv);
    if (status != kOk) return status;
    *context_out = context.release();
    return kOk;
  });
}

void evo_context_free(evo_context *context) { delete context; }
size_t evo_context_position(const evo_context *context) {
  return context == nullptr ? 0 : context->context->position();
}
size_t evo_context_capacity(const evo_context *context) {
  return context == nullptr ? 0 : context->context->context_capacity();
}
const char *evo_context_profile(const evo_context *context) {
  return context == nullptr ? "" : context->profile.c_str();
}

evo_status evo_context_prefill(evo_context *context, const evo_batch *batch,
                               evo_logits_callback callback, void *user_data) {
  return protect([&]() -> int {
    if (context == nullptr || batch == nullptr || callback == nullptr)
      return fail(evob::kInvalidArgument, "context, batch and callback are required");
    if (context->failed || context->context->poisoned())
      return fail(evob::kInvalidArgument, "context was invalidated by an earlier failure");
    if (context->context->position() != 0)
      return fail(evob::kInvalidArgument, "prefill requires a fresh context");
    std::vector<std::uint32_t> tokens;
    int status = single_sequence_tokens(batch, &tokens);
    if (status != kOk) return status;
    if (tokens.size() > context->context->context_capacity())
      return fail(evob::kInvalidArgument, "sequence exceeds the context capacity");
    context->failed = true;  // cleared only if every chunk and callback succeeds
    const std::size_t capacity = context->context->activation_capacity();
    const std::size_t columns = context->context->config().vocab;
    std::vector<float> logits;
    for (std::size_t offset = 0; offset < tokens.size();) {
      const std::size_t rows = std::min(capacity, tokens.size() - offset);
      const std::vector<std::uint32_t> chunk(tokens.begin() + offset, tokens.begin() + offset + rows);
      status = offset == 0 ? context->context->prefill(chunk, &logits)
                           : context->context->prefill_chunk(chunk, &logits);
      if (status != kOk) return status;
      if (logits.size() != rows * columns)
        return fail(evob::kInternal, "backend returned incomplete logits");
      const evo_status callback_status = callback(logits.data(), rows, columns, offset, user_data);
      if (callback_status != EVO_STATUS_OK)
        return fail(valid_status(callback_status) ? callback_status : EVO_STATUS_INTERNAL,
                    "logits consumer aborted prefill");
      offset += rows;
    }
    context->failed = false;
    return kOk;
  });
}

evo_status evo_context_decode(evo_context *context, uint32_t token, evo_logits_callback callback,
                              void *user_data) {
  return protect([&]() -> int {
    if (context == nullptr || callback == nullptr)
      return fail(evob::kInvalidArgument, "context and callback are required");
    if (context->failed || context->context->poisoned())
      return fail(evob::kInvalidArgument, "context was invalidated by an earlier failure");
    std::vector<float> logits;
    const std::size_t offset = context->context->position();
    int status = context->context->decode(token, &logits);
    if (status != kOk) {
      if (context->context->poisoned()) context->failed = true;
      return status;
    }
    const evo_status callback_status =
        callback(logits.data(), 1, context->context->config().vocab, offset, user_data);
    if (callback_status != EVO_STATUS_OK) {
      context->failed = true;
      return fail(valid_status(callback_status) ? callback_status : EVO_STATUS_INTERNAL,
                  "logits consumer aborted decode");
    }
    return kOk;
  });
}

// Shared body of evo_context_embed / evo_context_embed_ex (upstream src/c_api.cpp:1075-1330): a fresh
// context, one sequence, chunks of the activation capacity, the context advanced as by a prefill.
// `deliver` gets every chunk's rows (pooling "none") or the pooled row once at the end.
static int embed_chunks(evo_context *context, const evo_batch *batch, const size_t layer, const std::string &pooling,
                        const std::function<evo_status(const float *, size_t rows, size_t offset, size_t total)> &deliver) {
  if (context->failed || context->context->poisoned())
    return fail(evob::kInvalidArgument, "context was invalidated by an earlier failure");
  if (context->context->position() != 0)
    return fail(evob::kInvalidArgument, "embedding requires a fresh context");
  std::vector<std::uint32_t> tokens;
  int status = single_sequence_tokens(batch, &tokens);
  if (status != kOk) return status;
  if (tokens.size() > context->context->context_capacity())
    return fail(evob::kInvalidArgument, "sequence exceeds the context capacity");
  if (layer >= context->context->config().layers)
    return fail(evob::kInvalidArgument, "layer capture index or output is invalid");
  context->failed = true;  // cleared only if every chunk and callback succeeds
  const std::size_t capacity = context->context->activation_capacity();
  const std::size_t width = context->context->config().width;
  std::vector<float> hidden, pooled(pooling == "mean" ? width : 0, 0.0F);
  for (std::size_t offset = 0; offset < tokens.size();) {
    const std::size_t rows = std::min(capacity, tokens.size() - offset);
    const std::vector<std::uint32_t> chunk(tokens.begin() + offset, tokens.begin() + offset + rows);
    status = context->context->prefill_chunk_embedding(chunk, layer, offset == 0, &hidden);
    if (status != kOk) return status;
    if (hidden.size() != rows * width) return fail(evob::kInternal, "backend returned an incomplete embedding");
    if (pooling == "none") {
      const evo_status delivered = deliver(hidden.data(), rows, offset, tokens.size());
      if (delivered != EVO_STATUS_OK)
        return fail(valid_status(delivered) ? delivered : EVO_STATUS_INTERNAL, "embedding consumer aborted");
    } else if (pooling == "mean") {
      for (std::size_t r = 0; r < rows; ++r)
        for (std::size_t c = 0; c < width; ++c) pooled[c] += hidden[r * width + c];
    }
    offset += rows;
  }
  if (pooling != "none") {
    const float *row = pooled.data();
    if (pooling == "mean") {
      for (float &v : pooled) v /= static_cast<float>(tokens.size());
    } else {
      row = hidden.data() + (hidden.size() / width - 1) * width;  // "last": final row of the final chunk
    }
    const evo_status delivered = deliver(row, 1, 0, tokens.size());
    if (delivered != EVO_STATUS_OK)
      return fail(valid_status(delivered) ? delivered : EVO_STATUS_INTERNAL, "embedding consumer aborted");
  }
  context->failed = false;
  return kOk;
}

evo_status evo_context_embed(evo_context *context, const evo_batch *batch, size_t layer,
                             evo_embedding_callback callback, void *user_data) {
  return protect([&]() -> int {
    if (context == nullptr || batch == nullptr || callback == nullptr)
      return fail(evob::kInvalidArgument, "context, batch and callback are required");
    const std::size_t width = context->context->config().width;
    return embed_chunks(context, batch, layer, "none",
                        [&](const float *rows, size_t count, size_t offset, size_t) {
                          return callback(rows, count, width, offset, user_data);
                        });
  });
}

evo_status evo_context_embed_ex(evo_context *context, const evo_batch *batch,
                                const evo_embedding_options *options,
                                evo_embedding_ex_callback callback, void *user_data) {
  return protect([&]() -> int {
    if (context == nullptr || batch == nullptr || callback == nullptr)
      return fail(evob::kInvalidArgument, "context, batch and callback are required");
    evo_embedding_options chosen = evo_embedding_default_options();
    if (options != nullptr) {
      if (options->struct_size < sizeof(evo_embedding_options))
        return fail(evob::kInvalidArgument, "evo_embedding_options.struct_size is too small");
      chosen = *options;
    }
    if (chosen.preset != nullptr && chosen.preset[0] != '\0')
      return fail(evob::kUnsupported, "embedding presets are not defined for StripedHyena2");
    if (chosen.layer == static_cast<size_t>(-1))
      return fail(evob::kInvalidArgument, "explicit embedding requires layer");
    const std::string pooling = chosen.pooling == nullptr || chosen.pooling[0] == '\0' ? "none" : chosen.pooling;
    if (pooling != "none" && pooling != "mean" && pooling != "last")
      return fail(evob::kInvalidArgument, "pooling must be none, mean, or last");
    const std::size_t layer = chosen.layer;
    const std::size_t width = context->context->config().width;
    // unpooled rows are handed over once, after the last chunk (upstream collects them the same way)
    std::vector<float> collected;
    const auto once = [&](const float *rows, size_t count, size_t offset, size_t total) -> evo_status {
                          evo_embedding_result_info info{};
                          info.struct_size = sizeof(info);
                          info.resolved_preset = "";
                          info.hidden_tap = "explicit-layer";
                          info.pooling = pooling.c_str();
                          info.layer = layer;
                          info.original_length = info.effective_length = info.token_count = total;
                          info.rows = count;
                          info.columns = width;
                          return callback(rows, count, width, offset, &info, user_data);
    };
    return embed_chunks(context, batch, layer, pooling,
                        [&](const float *rows, size_t count, size_t offset, size_t total) -> evo_status {
                          if (pooling != "none") return once(rows, count, offset, total);
                          collected.insert(collected.end(), rows, rows + count * width);
                          if (offset + count < total) return EVO_STATUS_OK;
                          return once(collected.data(), total, 0, total);
                        });
  });
}

evo_status evo_batch_create(size_t sequence_capacity, evo_batch **batch_out) {
  return protect([&]() -> int {
    if (batch_out == nullptr || sequence_capacity == 0)
      return fail(evob::kInvalidArgument, "batch capacity and output are required");
    auto *batch = new evo_batch();
    batch->capacity = sequence_capacity;
    *batch_out = batch;
    return kOk;
  });
}
void evo_batch_free(evo_batch *batch) { delete batch; }
void evo_batch_clear(evo_batch *batch) {
  if (batch != nullptr) batch->sequences.clear();
}
evo_status evo_batch_add_sequence(evo_batch *batch, const uint8_t *sequence, size_t length) {
  return protect([&]() -> int {
    if (batch == nullptr || sequence == nullptr || length == 0)
      return fail(evob::kInvalidArgument, "batch and a non-empty sequence are required");
    if (batch->sequences.size() >= batch->capacity)
      return fail(evob::kInvalidArgument, "batch sequence capacity exceeded");
    batch->sequences.emplace_back(sequence, sequence + length);
    return kOk;
  });
}
size_t evo_batch_sequence_count(const evo_batch *batch) {
  return batch == nullptr ? 0 : batch->sequences.size();
}
size_t evo_batch_token_count(const evo_batch *batch) {
  size_t total = 0;
  if (batch != nullptr)
    for (const auto &s : batch->sequences) total += s.size();
  return total;
}

evo_status evo_sampler_create(const evo_sampler_params *params, evo_sampler **sampler_out) {
  return protect([&]() -> int {
    if (sampler_out == nullptr) return fail(evob::kInvalidArgument, "sampler output is required");
    *sampler_out = nullptr;
    evo_sampler_params p = evo_sampler_default_params();
    if (params != nullptr) {
      if (params->struct_size < sizeof(evo_sampler_params))
        return fail(evob::kInvalidArgument, "evo_sampler_params.struct_size is too small");
      p = *params;
    }
    evob::SamplingConfig config;
    config.temperature = p.temperature;
    config.top_k = p.top_k;
    config.top_p = p.top_p;
    config.seed = p.seed;
    const int status = evob::validate_sampling(config);
    if (status != kOk) return status;
    *sampler_out = new evo_sampler(config);
    return kOk;
  });
}
void evo_sampler_free(evo_sampler *sampler) { delete sampler; }
evo_status evo_sampler_sample(evo_sampler *sampler, const float *logits, size_t count,
                              uint32_t *token_out) {
  return protect([&]() -> int {
    if (sampler == nullptr) return fail(evob::kInvalidArgument, "sampler is required");
    return sampler->sampler.sample(logits, count, token_out);
  });
}

// ---- extensions (include/evo/evo_b200.h)
evo_status evo_b200_context_prefill_device(evo_context *context, const uint32_t *device_tokens,
                                           size_t rows, int stateless,
                                           const void **device_logits_out) {
  return protect([&]() -> int {
    if (context == nullptr) return fail(evob::kInvalidArgument, "context is required");
    if (context->failed || context->context->poisoned())
      return fail(evob::kInvalidArgument, "context was invalidated by an earlier failure");
    const int status = context->context->prefill_device(device_tokens, rows, stateless != 0);
    if (status != kOk) {
      context->failed = true;
      return status;
    }
    if (device_logits_out != nullptr) *device_logits_out = context->context->device_logits();
    return kOk;
  });
}

evo_status evo_b200_context_continue_device(evo_context *context, const uint32_t *device_tokens,
                                            size_t rows, const void **device_logits_out) {
  return protect([&]() -> int {
    if (context == nullptr) return fail(evob::kInvalidArgument, "context is required");
    if (context->failed || context->context->poisoned())
      return fail(evob::kInvalidArgument, "context was invalidated by an earlier failure");
    const int status = context->context->continue_device(device_tokens, rows);
    if (status != kOk) {
      if (context->context->poisoned()) context->failed = true;
      return status;
    }
    if (device_logits_out != nullptr) *device_logits_out = context->context->device_logits();
    return kOk;
  });
}

const char *evo_b200_dump_point_name(int32_t point) { return evob::dump_point_name(point); }

static int make_dump_plan(const evo_b200_dump_request *requests, size_t count, evo_b200_dump_callback callback,
                          void *user_data, evob::DumpPlan *plan) {
  if ((requests == nullptr && count != 0) || callback == nullptr)
    return fail(evob::kInvalidArgument, "dump requests and callback are required");
  for (size_t i = 0; i < count; ++i) {
    if (requests[i].point < 0 || requests[i].point >= EVO_B200_DUMP_POINT_COUNT)
      return fail(evob::kInvalidArgument, "dump point is out of range");
    plan->requests.push_back({requests[i].layer, static_cast<evob::DumpPoint>(requests[i].point)});
  }
  plan->sink = [callback, user_data](const evob::DumpPlan::Request &request, const float *values,
                                     std::size_t rows, std::size_t columns) -> int {
    const evo_status status =
        callback(request.layer, static_cast<int32_t>(request.point), values, rows, columns, user_data);
    return status == EVO_STATUS_OK ? kOk : (valid_status(status) ? status : EVO_STATUS_INTERNAL);
  };
  return kOk;
}

evo_status evo_b200_context_prefill_with_dumps(evo_context *context, const evo_batch *batch,
                                               const evo_b200_dump_request *requests, size_t request_count,
                                               int cached_attention, evo_b200_dump_callback dump_callback,
                                               evo_logits_callback logits_callback, void *user_data) {
  return protect([&]() -> int {
    if (context == nullptr || batch == nullptr || logits_callback == nullptr)
      return fail(evob::kInvalidArgument, "context, batch and callbacks are required");
    if (context->failed || context->context->poisoned())
      return fail(evob::kInvalidArgument, "context was invalidated by an earlier failure");
    evob::DumpPlan plan;
    int status = make_dump_plan(requests, request_count, dump_callback, user_data, &plan);
    if (status != kOk) return status;
    std::vector<std::uint32_t> tokens;
    status = single_sequence_tokens(batch, &tokens);
    if (status != kOk) return status;
    if (tokens.size() > context->context->activation_capacity())
      return fail(evob::kUnsupported, "a prefill with dumps must fit one activation chunk");
    context->failed = true;
    std::vector<float> logits;
    status = context->context->prefill_with_dumps(tokens, plan, cached_attention != 0, &logits);
    if (status != kOk) return status;
    const evo_status callback_status =
        logits_callback(logits.data(), tokens.size(), context->context->config().vocab, 0, user_data);
    if (callback_status != EVO_STATUS_OK)
      return fail(valid_status(callback_status) ? callback_status : EVO_STATUS_INTERNAL,
                  "logits consumer aborted prefill");
    context->failed = false;
    return kOk;
  });
}

evo_status evo_b200_context_decode_with_dumps(evo_context *context, uint32_t token,
                                              const evo_b200_dump_request *requests, size_t request_count,
                                              evo_b200_dump_callback dump_callback,
                                              evo_logits_callback logits_callback, void *user_data) {
  return protect([&]() -> int {
    if (context == nullptr || logits_callback == nullptr)
      return fail(evob::kInvalidArgument, "context and callbacks are required");
    if (context->failed || context->context->poisoned())
      return fail(evob::kInvalidArgument, "context was invalidated by an earlier failure");
    evob::DumpPlan plan;
    int status = make_dump_plan(requests, request_count, dump_callback, user_data, &plan);
    if (status != kOk) return status;
    std::vector<float> logits;
    const std::size_t offset = context->context->position();
    status = context->context->decode_with_dumps(token, plan, &logits);
    if (status != kOk) {
      if (context->context->poisoned()) context->failed = true;
      return status;
    }
    const evo_status callback_status =
        logits_callback(logits.data(), 1, context->context->config().vocab, offset, user_data);
    if (callback_status != EVO_STATUS_OK) {
      context->failed = true;
      return fail(valid_status(callback_status) ? callback_status : EVO_STATUS_INTERNAL,
                  "logits consumer aborted decode");
    }
    return kOk;
  });
}

evo_status evo_b200_variant_window_make(const char *sequence, size_t sequence_length, size_t position_1based,
                                        const char *reference, size_t reference_length, const char *alternate,
                                        size_t alternate_length, size_t maximum_tokens,
                                        evo_b200_variant_window *window, char *reference_window,
                                        char *alternate_window, size_t window_capacity) {
  return protect([&]() -> int {
    if (sequence == nullptr || reference == nullptr || alternate == nullptr || window == nullptr ||
        window->struct_size < sizeof(evo_b200_variant_window))
      return fail(evob::kInvalidArgument, "variant window arguments are invalid");
    evob::VariantWindow made;
    const int status = evob::make_variant_window({sequence, sequence_length}, position_1based,
                                                 {reference, reference_length}, {alternate, alternate_length},
                                                 maximum_tokens, &made);
    if (status != kOk) return status;
    if ((reference_window != nullptr || alternate_window != nullptr) &&
        window_capacity < std::max(made.reference.size(), made.alternate.size()))
      return fail(evob::kInvalidArgument, "variant window buffers are too small");
    window->reference_start = made.reference_start;
    window->reference_end = made.reference_end;
    window->variant_offset = made.variant_offset;
    window->reference_length = made.reference.size();
    window->alternate_length = made.alternate.size();
    if (reference_window != nullptr) std::memcpy(reference_window, made.reference.data(), made.reference.size());
    if (alternate_window != nullptr) std::memcpy(alternate_window, made.alternate.data(), made.alternate.size());
    return kOk;
  });
}

evo_status evo_b200_reverse_complement(const char *sequence, size_t length, char *output) {
  return protect([&]() -> int {
    if (sequence == nullptr || output == nullptr)
      return fail(evob::kInvalidArgument, "reverse-complement arguments are invalid");
    std::string reversed;
    const int status = evob::reverse_complement({sequence, length}, &reversed);
    if (status != kOk) return status;
    std::memcpy(output, reversed.data(), reversed.size());
    return kOk;
  });
}

evo_status evo_b200_vcf_stream(const char *path, evo_b200_vcf_callback callback, void *user_data) {
  return protect([&]() -> int {
    if (path == nullptr || callback == nullptr)
      return fail(evob::kInvalidArgument, "VCF path and callback are required");
    return evob::stream_vcf_file(path, [&](const evob::VcfRecord &record) -> int {
      evo_b200_vcf_record view{};
      view.struct_size = sizeof(view);
      view.contig = record.contig.c_str();
      view.id = record.id.c_str();
      view.reference = record.reference.c_str();
      view.alternate = record.alternate.c_str();
      view.position_1based = record.position_1based;
      view.record_index = record.record_index;
      view.allele_index = record.allele_index;
      view.line_number = record.line_number;
      const evo_status status = callback(&view, user_data);
      if (status == EVO_STATUS_OK) return kOk;
      return fail(valid_status(status) ? status : EVO_STATUS_INTERNAL, "VCF consumer stopped the stream");
    });
  });
}

evo_status evo_b200_reference_open(const char *path, evo_b200_reference **reference_out) {
  return protect([&]() -> int {
    if (reference_out != nullptr) *reference_out = nullptr;
    if (path == nullptr || reference_out == nullptr)
      return fail(evob::kInvalidArgument, "reference path and output are required");
    evob::ReferenceFasta *fasta = nullptr;
    const int status = evob::ReferenceFasta::open(path, &fasta);
    if (status != kOk) return status;
    auto *handle = new evo_b200_reference();
    handle->fasta.reset(fasta);
    *reference_out = handle;
    return kOk;
  });
}

void evo_b200_reference_free(evo_b200_reference *reference) { delete reference; }

evo_status evo_b200_reference_window(const evo_b200_reference *reference, const char *contig,
                                     size_t position_1based, const char *reference_allele,
                                     size_t reference_length, const char *alternate_allele,
                                     size_t alternate_length, size_t maximum_tokens, size_t *start, size_t *end,
                                     size_t *contig_length, char *sequence, size_t capacity) {
  return protect([&]() -> int {
    if (reference == nullptr || contig == nullptr || reference_allele == nullptr || alternate_allele == nullptr)
      return fail(evob::kInvalidArgument, "reference window arguments are invalid");
    evob::ReferenceSlice slice;
    const int status = reference->fasta->slice(contig, position_1based, {reference_allele, reference_length},
                                               {alternate_allele, alternate_length}, maximum_tokens, &slice);
    if (status != kOk) return status;
    if (sequence != nullptr && capacity < slice.sequence.size())
      return fail(evob::kInvalidArgument, "reference window buffer is too small");
    if (start != nullptr) *start = slice.start;
    if (end != nullptr) *end = slice.end;
    if (contig_length != nullptr) *contig_length = slice.contig_length;
    if (sequence != nullptr) std::memcpy(sequence, slice.sequence.data(), slice.sequence.size());
    return kOk;
  });
}

evo_status evo_b200_scheduler_create(const evo_model *model, const evo_b200_scheduler_params *params,
                                     evo_b200_scheduler **scheduler_out) {
  return protect([&]() -> int {
    if (scheduler_out != nullptr) *scheduler_out = nullptr;
    if (model == nullptr || params == nullptr || scheduler_out == nullptr ||
        params->struct_size < sizeof(evo_b200_scheduler_params))
      return fail(evob::kInvalidArgument, "model, scheduler parameters and output are required");
    const bool q8_kv = (params->context_flags & EVO_CONTEXT_FLAG_FAST_Q8_KV) != 0;
    const bool fp8_ffn = (params->context_flags & EVO_CONTEXT_FLAG_B200_FP8_FFN) != 0;
    const bool tensor_core = fp8_ffn || (params->context_flags & EVO_CONTEXT_FLAG_B200_TENSORCORE_FP8) != 0;
    auto handle = std::make_unique<evo_b200_scheduler>();
    const int status = evob::Scheduler::create(
        model->weights, params->workers, params->maximum_queue, params->context_size,
        fp8_ffn       ? evob::ExecutionProfile::kTensorCoreFfn
        : tensor_core ? evob::ExecutionProfile::kTensorCore
                      : evob::ExecutionProfile::kExact,
        (params->context_flags & EVO_CONTEXT_FLAG_B200_FULL_ARENA) != 0, q8_kv, &handle->scheduler);
    if (status != kOk) return status;
    *scheduler_out = handle.release();
    return kOk;
  });
}

void evo_b200_scheduler_free(evo_b200_scheduler *scheduler) { delete scheduler; }

evo_status evo_b200_scheduler_submit(evo_b200_scheduler *scheduler, const evo_b200_request *request,
                                     evo_b200_request_callback done, void *user_data, uint64_t *ticket) {
  return protect([&]() -> int {
    if (ticket != nullptr) *ticket = 0;
    if (scheduler == nullptr || request == nullptr || ticket == nullptr ||
        request->struct_size < sizeof(evo_b200_request) || (request->sequence == nullptr && request->length != 0))
      return fail(evob::kInvalidArgument, "scheduler, request and ticket output are required");
    if (request->kind != EVO_B200_REQUEST_SCORE && request->kind != EVO_B200_REQUEST_GENERATE)
      return fail(evob::kInvalidArgument, "request kind must be score or generate");
    evob::SchedulerRequest copy;
    copy.kind = request->kind == EVO_B200_REQUEST_SCORE ? evob::SchedulerRequest::Kind::kScore
                                                        : evob::SchedulerRequest::Kind::kGenerate;
    copy.sequence.assign(request->sequence, request->sequence + request->length);
    copy.new_tokens = request->new_tokens;
    if (copy.kind == evob::SchedulerRequest::Kind::kGenerate) {
      copy.sampling.temperature = request->sampler.temperature;
      copy.sampling.top_k = request->sampler.top_k;
      copy.sampling.top_p = request->sampler.top_p;
      copy.sampling.seed = request->sampler.seed;
    }
    *ticket = scheduler->scheduler->submit(
        std::move(copy), [done, user_data](const std::uint64_t id, const evob::SchedulerResult &result) {
          if (done == nullptr) return;
          evo_b200_request_result view{};
          view.struct_size = sizeof(view);
          view.status = static_cast<evo_status>(result.status);
          view.error = result.error.c_str();
          view.cancelled = result.cancelled ? 1 : 0;
          view.log_likelihood = result.log_likelihood;
          view.scored_tokens = result.scored_tokens;
          view.token_log_likelihoods = result.token_log_likelihoods.data();
          view.generated = result.generated.data();
          view.generated_length = result.generated.size();
          view.queue_seconds = result.queue_seconds;
          view.run_seconds = result.run_seconds;
          done(id, &view, user_data);
        });
    return kOk;
  });
}

int evo_b200_scheduler_cancel(evo_b200_scheduler *scheduler, uint64_t ticket) {
  return scheduler != nullptr && scheduler->scheduler->cancel(ticket) ? 1 : 0;
}

evo_status evo_b200_scheduler_read_metrics(const evo_b200_scheduler *scheduler,
                                           evo_b200_scheduler_metrics *metrics) {
  return protect([&]() -> int {
    if (scheduler == nullptr || metrics == nullptr || metrics->struct_size < sizeof(evo_b200_scheduler_metrics))
      return fail(evob::kInvalidArgument, "scheduler and metrics output are required");
    const evob::SchedulerMetrics m = scheduler->scheduler->metrics();
    metrics->submitted = m.submitted;
    metrics->rejected = m.rejected;
    metrics->completed = m.completed;
    metrics->failed = m.failed;
    metrics->cancelled = m.cancelled;
    metrics->queued = m.queued;
    metrics->queue_peak = m.queue_peak;
    metrics->active = m.active;
    metrics->active_peak = m.active_peak;
    return kOk;
  });
}

void evo_b200_scheduler_wait_idle(const evo_b200_scheduler *scheduler) {
  if (scheduler != nullptr) scheduler->scheduler->wait_idle();
}

void *evo_b200_context_stream(const evo_context *context) {
  return context == nullptr ? nullptr : context->context->first_stream();
}

evo_status evo_b200_context_synchronize(evo_context *context) {
  return protect([&]() -> int {
    if (context == nullptr) return fail(evob::kInvalidArgument, "context is required");
    const int status = context->context->synchronize();
    if (status != kOk) context->failed = true;
    return status;
  });
}

evo_status evo_b200_context_profile_enable(evo_context *context, int enabled) {
  return protect([&]() -> int {
    if (context == nullptr) return fail(evob::kInvalidArgument, "context is required");
    context->context->set_profiling(enabled != 0);
    return kOk;
  });
}

size_t evo_b200_context_profile_read(const evo_context *context, double *milliseconds,
                                     uint64_t *launches, size_t capacity) {
  if (context == nullptr) return 0;
  double ms[evob::kProfileCategories];
  std::uint64_t counts[evob::kProfileCategories];
  context->context->read_profile(ms, counts);
  for (size_t i = 0; i < capacity && i < static_cast<size_t>(evob::kProfileCategories); ++i) {
    if (milliseconds != nullptr) milliseconds[i] = ms[i];
    if (launches != nullptr) launches[i] = counts[i];
  }
  return evob::kProfileCategories;
}

const char *evo_b200_profile_category_name(size_t index) {
  return evob::profile_category_name(static_cast<int>(index));
}

evo_status evo_b200_plan_stages(const size_t *layer_bytes, size_t layers, size_t stages,
                                int even_split, size_t *begins, size_t *ends) {
  return protect([&]() -> int {
    if (layer_bytes == nullptr || begins == nullptr || ends == nullptr || stages == 0 ||
        stages > 8 || layers < stages)
      return fail(evob::kInvalidArgument, "stage plan needs 1..8 stages and a layer per stage");
    const auto plan = evob::plan_stages(std::vector<std::size_t>(layer_bytes, layer_bytes + layers),
                                        stages, even_split != 0);
    if (plan.size() != stages) return fail(evob::kInternal, "stage planning failed");
    for (size_t i = 0; i < stages; ++i) {
      begins[i] = plan[i].first;
      ends[i] = plan[i].second;
    }
    return kOk;
  });
}

size_t evo_b200_context_stage_count(const evo_context *context) {
  return context == nullptr ? 0 : context->context->stages().size();
}

evo_status evo_b200_context_prefill_tokens(evo_context *context, const uint32_t *tokens, size_t token_count,
                                           int32_t mode, evo_logits_callback callback, void *user_data) {
  return protect([&]() -> int {
    if (context == nullptr || tokens == nullptr || token_count == 0 || callback == nullptr)
      return fail(evob::kInvalidArgument, "context, tokens and callback are required");
    if (mode < EVO_B200_PREFILL_FRESH || mode > EVO_B200_PREFILL_CHUNK)
      return fail(evob::kInvalidArgument, "unknown prefill mode");
    if (context->failed || context->context->poisoned())
      return fail(evob::kInvalidArgument, "context was invalidated by an earlier failure");
    evob::Context &model = *context->context;
    const std::size_t capacity = model.activation_capacity();
    const std::size_t columns = model.config().vocab;
    const std::size_t begin = mode == EVO_B200_PREFILL_CHUNK ? model.position() : 0;
    if (token_count > model.context_capacity() - std::min(begin, model.context_capacity()))
      return fail(evob::kInvalidArgument, "sequence exceeds the context capacity");
    if (mode != EVO_B200_PREFILL_FRESH && token_count > capacity)
      return fail(evob::kInvalidArgument, "this prefill form takes at most one activation chunk of tokens");
    std::vector<float> logits;
    for (std::size_t offset = 0; offset < token_count;) {
      const std::size_t rows = std::min(capacity, token_count - offset);
      const std::vector<std::uint32_t> chunk(tokens + offset, tokens + offset + rows);
      int status;
      switch (mode) {
        case EVO_B200_PREFILL_STATELESS: status = model.prefill_stateless(chunk, &logits); break;
        case EVO_B200_PREFILL_CACHED: status = model.prefill_cached(chunk, &logits); break;
        case EVO_B200_PREFILL_CHUNK: status = model.prefill_chunk(chunk, &logits); break;
        default: status = offset == 0 ? model.prefill(chunk, &logits) : model.prefill_chunk(chunk, &logits); break;
      }
      if (status != kOk) {
        if (model.poisoned()) context->failed = true;
        return status;
      }
      if (logits.size() != rows * columns) return fail(evob::kInternal, "backend returned incomplete logits");
      const evo_status callback_status = callback(logits.data(), rows, columns, begin + offset, user_data);
      if (callback_status != EVO_STATUS_OK) {
        context->failed = true;
        return fail(valid_status(callback_status) ? callback_status : EVO_STATUS_INTERNAL,
                    "logits consumer aborted prefill");
      }
      offset += rows;
    }
    return kOk;
  });
}

evo_status evo_b200_context_embed_tokens(evo_context *context, const uint32_t *tokens, size_t token_count, size_t layer,
                                         int32_t first_chunk, evo_embedding_callback callback, void *user_data) {
  return protect([&]() -> int {
    if (context == nullptr || tokens == nullptr || token_count == 0 || callback == nullptr)
      return fail(evob::kInvalidArgument, "context, tokens and callback are required");
    if (context->failed || context->context->poisoned())
      return fail(evob::kInvalidArgument, "context was invalidated by an earlier failure");
    evob::Context &model = *context->context;
    if (token_count > model.activation_capacity())
      return fail(evob::kInvalidArgument, "an embedding chunk takes at most one activation chunk of tokens");
    const std::size_t begin = first_chunk != 0 ? 0 : model.position();
    if (token_count > model.context_capacity() - std::min(begin, model.context_capacity()))
      return fail(evob::kInvalidArgument, "sequence exceeds the context capacity");
    const std::vector<std::uint32_t> chunk(tokens, tokens + token_count);
    std::vector<float> hidden;
    const int status = model.prefill_chunk_embedding(chunk, layer, first_chunk != 0, &hidden);
    if (status != kOk) {
      if (model.poisoned()) context->failed = true;
      return status;
    }
    const std::size_t width = model.config().width;
    if (hidden.size() != token_count * width) return fail(evob::kInternal, "backend returned an incomplete embedding");
    const evo_status delivered = callback(hidden.data(), token_count, width, begin, user_data);
    if (delivered != EVO_STATUS_OK) {
      context->failed = true;
      return fail(valid_status(delivered) ? delivered : EVO_STATUS_INTERNAL, "embedding consumer aborted");
    }
    return kOk;
  });
}

size_t evo_b200_context_activation_capacity(const evo_context *context) {
  return context == nullptr ? 0 : context->context->activation_capacity();
}

evo_status evo_b200_read_model_config(const char *path, int32_t allow_test_fixture, evo_b200_model_config *config,
                                      uint8_t *mixer_types, size_t mixer_capacity) {
  return protect([&]() -> int {
    if (path == nullptr || config == nullptr || config->struct_size < sizeof(evo_b200_model_config))
      return fail(evob::kInvalidArgument, "model path and a sized configuration struct are required");
    std::shared_ptr<evob::ModelFile> file;
    int status = evob::ModelFile::open(path, &file);
    if (status != kOk) return status;
    evob::ModelConfig c;
    status = evob::read_model_config(*file, allow_test_fixture != 0, &c);
    if (status != kOk) return status;
    status = evob::check_tensor_set(*file, c);
    if (status != kOk) return status;
    const auto copy_text = [](char (&target)[64], const std::string &source) {
      std::memset(target, 0, sizeof(target));
      std::memcpy(target, source.data(), std::min(source.size(), sizeof(target) - 1));
    };
    const std::size_t struct_size = config->struct_size;
    std::memset(config, 0, sizeof(*config));
    config->struct_size = struct_size;
    copy_text(config->model_id, c.model_id);
    copy_text(config->architecture, c.architecture);
    copy_text(config->artifact_profile, c.artifact_profile);
    config->vocab_size = c.vocab;
    config->width = c.width;
    config->layers = c.layers;
    config->heads = c.heads;
    config->state_size = c.state_size;
    config->inner_width = c.inner_width;
    config->short_filter_length = c.short_taps;
    config->hcs_filter_length = c.hcs_taps;
    config->hcm_filter_length = c.hcm_taps;
    config->hcs_filter_groups = c.hcs_groups;
    config->hcm_filter_groups = c.hcm_groups;
    config->max_seqlen = c.max_seqlen;
    config->epsilon = c.epsilon;
    config->rope_scale = c.rope_scale;
    config->rope_base = c.rope_base;
    config->qkv_source_head_major = c.qkv_source_head_major ? 1 : 0;
    config->hyena_projection_e4m3 = c.fp8_projection ? 1 : 0;
    config->hcm_filter_f32 = c.hcm_filter_f32 ? 1 : 0;
    config->test_fixture = c.test_fixture ? 1 : 0;
    if (mixer_types != nullptr)
      for (std::size_t i = 0; i < c.mixers.size() && i < mixer_capacity; ++i)
        mixer_types[i] = static_cast<uint8_t>(c.mixers[i]);
    return kOk;
  });
}

evo_status evo_b200_context_stage_info(const evo_context *context, size_t index,
                                       evo_b200_stage_info *info) {
  return protect([&]() -> int {
    if (context == nullptr || info == nullptr || info->struct_size < sizeof(evo_b200_stage_info))
      return fail(evob::kInvalidArgument, "stage query arguments are invalid");
    const auto stages = context->context->stages();
    if (index >= stages.size()) return fail(evob::kInvalidArgument, "stage index is out of range");
    info->device = stages[index].device;
    info->layer_begin = stages[index].layer_begin;
    info->layer_end = stages[index].layer_end;
    info->weight_bytes = stages[index].weight_bytes;
    info->cache_bytes = stages[index].cache_bytes;
    info->arena_bytes = stages[index].arena_bytes;
    return kOk;
  });
}

evo_status evo_b200_model_load_slice(const char *path, int32_t device, size_t slice_index,
                                     size_t slice_count, uint32_t flags, evo_model **model_out) {
  return protect([&]() -> int {
    if (model_out != nullptr) *model_out = nullptr;
    if (path == nullptr || model_out == nullptr)
      return fail(evob::kInvalidArgument, "model path and output are required");
    if (slice_count < 2)
      return fail(evob::kInvalidArgument, "a sliced pipeline has at least two slices; use evo_model_load");
    auto model = std::make_unique<evo_model>();
    int status = evob::ModelFile::open(path, &model->file);
    if (status != kOk) return status;
    status = evob::load_weights(*model->file, {device},
                                (flags & EVO_MODEL_FLAG_TEST_ONLY_ALLOW_SYNTHETIC) != 0, 0,
                                &model->weights, slice_index, slice_count);
    if (status != kOk) return status;
    *model_out = model.release();
    return kOk;
  });
}

static evo_status slice_call(evo_context *context, const std::function<int(evob::Context &)> &call) {
  return protect([&]() -> int {
    if (context == nullptr) return fail(evob::kInvalidArgument, "context is required");
    if (context->failed || context->context->poisoned())
      return fail(evob::kInvalidArgument, "context was invalidated by an earlier failure");
    const int status = call(*context->context);
    if (status != kOk && context->context->poisoned()) context->failed = true;
    return status;
  });
}

evo_status evo_b200_context_slice_embed(evo_context *context, const uint32_t *device_tokens,
                                        size_t row_begin, size_t rows) {
  return slice_call(context, [&](evob::Context &c) { return c.slice_embed(device_tokens, row_begin, rows); });
}
evo_status evo_b200_context_slice_run(evo_context *context, size_t row_begin, size_t rows) {
  return slice_call(context, [&](evob::Context &c) { return c.slice_run(row_begin, rows); });
}
evo_status evo_b200_context_slice_head(evo_context *context, size_t row_begin, size_t rows,
                                       const void **device_logits_out) {
  return slice_call(context, [&](evob::Context &c) {
    const int status = c.slice_head(row_begin, rows);
    if (status == kOk && device_logits_out != nullptr) *device_logits_out = c.device_logits();
    return status;
  });
}
void *evo_b200_context_slice_hidden(const evo_context *context) {
  return context == nullptr ? nullptr : context->context->slice_hidden();
}

}  // extern "C"
