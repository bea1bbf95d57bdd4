// evo::cuda model classes (upstream include/evo/cuda/model.hpp:16-229: RuntimeModelConfig readers,
// SingleGpuModel, PipelineModel) on this build's model-level C ABI (include/evo/evo.h and
// include/evo/evo_b200.h, libevo.so); see compat_common.hpp for what the layer is.
//
// How the pieces map:
//  * A model object owns one evo_model (the immutable device weights, shared between objects made by
//    initialize_shared) and one evo_context (caches, arena, streams).
//  * upstream's ModelFile does not expose the path it was opened from and the C ABI loads by path, so
//    the path is recovered from the process's table of memory mappings: the mapping that holds the
//    file's first tensor.  Single-file artifacts only.
//  * The configuration comes from evo_b200_read_model_config (same keys, same refusals); the exact-
//    support gate is upstream's own registry function, which stays part of upstream's core library.
//  * Layer dumps are written as NPY version 1.0 files of F32 [rows, columns], as upstream writes them.
//  * layer_limit, prefill_prefix / prefill_chunk_prefix / decode_prefix (the hybrid CLI's truncated
//    forward passes) are not offered by the C ABI and report `unsupported`.
#include "compat_common.hpp"

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <memory>
#include <sstream>
#include <utility>

#include "evo/cuda/model.hpp"
#include "evo/model_registry.hpp"

#include "../../include/evo/evo.h"
#include "../../include/evo/evo_b200.h"

namespace evo::cuda {

using evo_b200_compat::invalid;

namespace {

Status from_abi(const evo_status status, const char *operation) {
  if (status == EVO_STATUS_OK) return Status::Ok();
  std::string message = operation;
  const char *detail = evo_last_error();
  if (detail != nullptr && detail[0] != '\0') {
    message += ": ";
    message += detail;
  }
  ErrorCode code = ErrorCode::kInternal;
  switch (status) {
    case EVO_STATUS_INVALID_ARGUMENT: code = ErrorCode::kInvalidArgument; break;
    case EVO_STATUS_IO: code = ErrorCode::kIo; break;
    case EVO_STATUS_MODEL_FORMAT: code = ErrorCode::kModelFormat; break;
    case EVO_STATUS_UNSUPPORTED: code = ErrorCode::kUnsupported; break;
    case EVO_STATUS_CUDA: code = ErrorCode::kCuda; break;
    default: break;
  }
  return {code, message};
}

// Path of the file mapped at `address`, from /proc/self/maps ("" when there is none).
std::string mapped_path(const void *address) {
  std::ifstream maps("/proc/self/maps");
  const auto wanted = reinterpret_cast<std::uintptr_t>(address);
  std::string line;
  while (std::getline(maps, line)) {
    unsigned long long begin = 0, end = 0;
    int consumed = 0;
    // begin-end perms offset dev inode path
    if (std::sscanf(line.c_str(), "%llx-%llx %*s %*s %*s %*s %n", &begin, &end, &consumed) < 2) continue;
    if (wanted < begin || wanted >= end || consumed <= 0 || static_cast<std::size_t>(consumed) >= line.size()) continue;
    std::string path = line.substr(static_cast<std::size_t>(consumed));
    const std::string deleted = " (deleted)";
    if (path.size() > deleted.size() && path.compare(path.size() - deleted.size(), deleted.size(), deleted) == 0)
      path.resize(path.size() - deleted.size());
    return path.empty() || path[0] != '/' ? std::string() : path;
  }
  return {};
}

Status path_of(const ModelFile &model, std::string *path) {
  if (model.tensors().empty()) return invalid("the model file is not open");
  if (model.shard_count() > 1)
    return {ErrorCode::kUnsupported, "sharded artifacts are loaded through the C ABI by path, not through a ModelFile"};
  const auto *const data = model.tensor_data(model.tensors().front());
  *path = data == nullptr ? std::string() : mapped_path(data);
  if (path->empty()) return {ErrorCode::kIo, "cannot find the path the model file was mapped from"};
  return Status::Ok();
}

Status read_config(const std::string &path, const bool allow_test_fixture, RuntimeModelConfig *config) {
  evo_b200_model_config raw{};
  raw.struct_size = sizeof(raw);
  std::vector<std::uint8_t> mixers(4096, 0);
  auto status = from_abi(evo_b200_read_model_config(path.c_str(), allow_test_fixture ? 1 : 0, &raw, mixers.data(),
                                                    mixers.size()),
                         "read the runtime model configuration");
  if (!status.ok()) return status;
  if (raw.layers > mixers.size()) return {ErrorCode::kUnsupported, "more blocks than the layer can describe"};
  RuntimeModelConfig c;
  c.model_id = raw.model_id;
  c.architecture = raw.architecture;
  c.artifact_profile = raw.artifact_profile;
  c.vocab_size = raw.vocab_size;
  c.width = raw.width;
  c.layers = raw.layers;
  c.heads = raw.heads;
  c.state_size = raw.state_size;
  c.inner_width = raw.inner_width;
  c.short_filter_length = raw.short_filter_length;
  c.hcs_filter_length = raw.hcs_filter_length;
  c.hcm_filter_length = raw.hcm_filter_length;
  c.hcs_filter_groups = raw.hcs_filter_groups;
  c.hcm_filter_groups = raw.hcm_filter_groups;
  c.hcl_filter_groups = raw.width;  // one long filter per channel
  c.max_seqlen = raw.max_seqlen;
  c.epsilon = raw.epsilon;
  c.rope_scale = raw.rope_scale;
  c.rope_base = raw.rope_base;
  c.interpolated_rope = raw.rope_scale != 1.0F;
  c.qkv_head_major = false;  // the runtime re-orders a head-major checkpoint when it loads it
  c.qkv_source_head_major = raw.qkv_source_head_major != 0;
  c.hyena_projection_dtype = raw.hyena_projection_e4m3 != 0 ? HyenaProjectionDType::kE4M3Sw : HyenaProjectionDType::kBF16;
  c.hcm_filter_dtype = raw.hcm_filter_f32 != 0 ? HcmFilterDType::kF32 : HcmFilterDType::kBF16;
  c.test_fixture = raw.test_fixture != 0;
  c.mixer_types.reserve(raw.layers);
  for (std::size_t i = 0; i < raw.layers; ++i) {
    switch (mixers[i]) {
      case 0: c.mixer_types.push_back(MixerType::kHcs); break;
      case 1: c.mixer_types.push_back(MixerType::kHcm); break;
      case 2: c.mixer_types.push_back(MixerType::kHcl); break;
      default: c.mixer_types.push_back(MixerType::kAttention); break;
    }
  }
  *config = std::move(c);
  return Status::Ok();
}

struct ModelHandle final {
  evo_model *model{nullptr};
  ~ModelHandle() { evo_model_free(model); }
};

// What both model classes are made of.
struct Core final {
  std::shared_ptr<ModelHandle> weights;
  evo_context *context{nullptr};
  RuntimeModelConfig config;
  std::vector<StageAssignment> stages;
  std::vector<int> devices;
  bool q8{false};

  ~Core() { evo_context_free(context); }

  Status make_context(const std::size_t context_capacity, const InferenceProfile profile) {
    if (profile != InferenceProfile::kExact && profile != InferenceProfile::kFastQ8Kv)
      return {ErrorCode::kUnsupported, "the CUDA backend runs the exact and fast-q8-kv profiles"};
    evo_context_params params = evo_context_default_params();
    params.context_size = context_capacity;
    params.flags = profile == InferenceProfile::kFastQ8Kv ? static_cast<std::uint32_t>(EVO_CONTEXT_FLAG_FAST_Q8_KV) : 0U;
    evo_context_free(context);
    context = nullptr;
    auto status = from_abi(evo_context_create(weights->model, &params, &context), "create the CUDA context");
    if (!status.ok()) return status;
    q8 = profile == InferenceProfile::kFastQ8Kv;
    config.inference_profile = profile;
    refresh_stages();
    return Status::Ok();
  }

  void refresh_stages() {
    stages.clear();
    if (context == nullptr) return;
    const std::size_t count = evo_b200_context_stage_count(context);
    for (std::size_t index = 0; index < count; ++index) {
      evo_b200_stage_info info{};
      info.struct_size = sizeof(info);
      if (evo_b200_context_stage_info(context, index, &info) != EVO_STATUS_OK) break;
      stages.push_back({info.device, info.layer_begin, info.layer_end, info.weight_bytes, info.cache_bytes,
                        info.arena_bytes});
    }
  }

  Status load(const ModelFile &file, const std::vector<int> &device_list, const std::size_t context_capacity,
              const bool allow_test_fixture, const InferenceProfile profile, const std::size_t layer_limit) {
    std::string path;
    auto status = path_of(file, &path);
    if (!status.ok()) return status;
    RuntimeModelConfig candidate;
    status = read_config(path, allow_test_fixture, &candidate);
    if (!status.ok()) return status;
    status = validate_runtime_exact_support(candidate, profile);
    if (!status.ok()) return status;
    if (layer_limit != 0 && layer_limit != candidate.layers)
      return {ErrorCode::kUnsupported, "a layer limit is not available through the C ABI"};
    if (device_list.empty()) return invalid("at least one CUDA device is required");
    std::vector<std::int32_t> ids(device_list.begin(), device_list.end());
    evo_model_params params = evo_model_default_params();
    params.backend = EVO_BACKEND_CUDA;
    params.devices = ids.data();
    params.device_count = ids.size();
    params.flags = allow_test_fixture ? static_cast<std::uint32_t>(EVO_MODEL_FLAG_TEST_ONLY_ALLOW_SYNTHETIC) : 0U;
    auto handle = std::make_shared<ModelHandle>();
    status = from_abi(evo_model_load(path.c_str(), &params, &handle->model), "load the model onto the CUDA devices");
    if (!status.ok()) return status;
    weights = std::move(handle);
    config = std::move(candidate);
    devices = device_list;
    return make_context(context_capacity, profile);
  }

  // ---- passes
  struct Rows final {
    std::vector<float> *values;
    std::size_t columns{0};
  };
  static evo_status gather(const float *values, const std::size_t rows, const std::size_t columns, std::size_t,
                           void *user_data) {
    auto *const target = static_cast<Rows *>(user_data);
    target->columns = columns;
    target->values->insert(target->values->end(), values, values + rows * columns);
    return EVO_STATUS_OK;
  }

  Status ready(const void *output) const {
    if (context == nullptr) return invalid("the model is not loaded");
    if (output == nullptr) return invalid("the output vector is null");
    return Status::Ok();
  }

  Status prefill(const std::vector<TokenId> &tokens, const int mode, std::vector<float> *logits, const char *what) {
    auto status = ready(logits);
    if (!status.ok()) return status;
    if (tokens.empty()) return invalid("a prefill needs at least one token");
    logits->clear();
    Rows rows{logits};
    return from_abi(evo_b200_context_prefill_tokens(context, tokens.data(), tokens.size(), mode, &Core::gather, &rows), what);
  }

  Status decode(const TokenId token, std::vector<float> *logits) {
    auto status = ready(logits);
    if (!status.ok()) return status;
    logits->clear();
    Rows rows{logits};
    return from_abi(evo_context_decode(context, token, &Core::gather, &rows), "cached decode");
  }

  // ---- dumps
  struct DumpJob final {
    const std::vector<LayerDump> *dumps;
    Rows logits;
    std::string error;
  };
  static bool write_npy(const std::string &path, const float *values, const std::size_t rows, const std::size_t columns) {
    std::ostringstream shape;
    shape << "{'descr': '<f4', 'fortran_order': False, 'shape': (" << rows << ", " << columns << "), }";
    std::string header = shape.str();
    // magic (6) + version (2) + length (2) + header, padded with spaces to a multiple of 64, newline last
    const std::size_t unpadded = 10 + header.size() + 1;
    header.append((64 - unpadded % 64) % 64, ' ');
    header.push_back('\n');
    std::ofstream out(path, std::ios::binary | std::ios::trunc);
    if (!out) return false;
    const unsigned char preamble[10] = {0x93, 'N', 'U', 'M', 'P', 'Y', 1, 0,
                                        static_cast<unsigned char>(header.size() & 0xffU),
                                        static_cast<unsigned char>((header.size() >> 8U) & 0xffU)};
    out.write(reinterpret_cast<const char *>(preamble), sizeof(preamble));
    out.write(header.data(), static_cast<std::streamsize>(header.size()));
    out.write(reinterpret_cast<const char *>(values), static_cast<std::streamsize>(rows * columns * sizeof(float)));
    return static_cast<bool>(out);
  }
  static evo_status on_dump(const std::size_t layer, const std::int32_t point, const float *values, const std::size_t rows,
                            const std::size_t columns, void *user_data) {
    auto *const job = static_cast<DumpJob *>(user_data);
    for (const LayerDump &dump : *job->dumps) {
      if (dump.layer != layer || static_cast<std::int32_t>(dump.point) != point) continue;
      if (!write_npy(dump.path, values, rows, columns)) {
        job->error = "cannot write the layer dump " + dump.path;
        return EVO_STATUS_IO;
      }
    }
    return EVO_STATUS_OK;
  }
  static evo_status on_dump_logits(const float *values, const std::size_t rows, const std::size_t columns,
                                   const std::size_t offset, void *user_data) {
    return gather(values, rows, columns, offset, &static_cast<DumpJob *>(user_data)->logits);
  }

  Status requests_of(const std::vector<LayerDump> &dumps, std::vector<evo_b200_dump_request> *requests) const {
    for (const LayerDump &dump : dumps) {
      const auto point = static_cast<std::int32_t>(dump.point);
      if (dump.path.empty() || dump.layer >= config.layers || point < 0 || point >= EVO_B200_DUMP_POINT_COUNT)
        return invalid("a layer dump names no path, a block outside the model or an unknown point");
      const bool seen = std::any_of(requests->begin(), requests->end(), [&](const evo_b200_dump_request &r) {
        return r.layer == dump.layer && r.point == point;
      });
      if (!seen) requests->push_back({dump.layer, point});
    }
    return Status::Ok();
  }

  Status prefill_with_dumps(const std::vector<TokenId> &tokens, std::vector<float> *logits,
                            const std::vector<LayerDump> &dumps, const bool cached) {
    if (dumps.empty())
      return prefill(tokens, cached ? EVO_B200_PREFILL_CACHED : EVO_B200_PREFILL_FRESH, logits, "prefill");
    auto status = ready(logits);
    if (!status.ok()) return status;
    std::vector<evo_b200_dump_request> requests;
    status = requests_of(dumps, &requests);
    if (!status.ok()) return status;
    std::vector<std::uint8_t> bytes;
    bytes.reserve(tokens.size());
    for (const TokenId token : tokens) {
      if (token > 0xffU) return invalid("byte-level models take token ids below 256");
      bytes.push_back(static_cast<std::uint8_t>(token));
    }
    if (bytes.empty()) return invalid("a prefill needs at least one token");
    evo_batch *batch = nullptr;
    status = from_abi(evo_batch_create(1, &batch), "create a batch");
    if (!status.ok()) return status;
    status = from_abi(evo_batch_add_sequence(batch, bytes.data(), bytes.size()), "add the sequence");
    logits->clear();
    DumpJob job{&dumps, Rows{logits}, {}};
    if (status.ok())
      status = from_abi(evo_b200_context_prefill_with_dumps(context, batch, requests.data(), requests.size(),
                                                            cached ? 1 : 0, &Core::on_dump, &Core::on_dump_logits, &job),
                        "prefill with layer dumps");
    evo_batch_free(batch);
    if (!status.ok() && !job.error.empty()) return {ErrorCode::kIo, job.error};
    return status;
  }

  Status decode_with_dumps(const TokenId token, std::vector<float> *logits, const std::vector<LayerDump> &dumps) {
    if (dumps.empty()) return decode(token, logits);
    auto status = ready(logits);
    if (!status.ok()) return status;
    std::vector<evo_b200_dump_request> requests;
    status = requests_of(dumps, &requests);
    if (!status.ok()) return status;
    logits->clear();
    DumpJob job{&dumps, Rows{logits}, {}};
    status = from_abi(evo_b200_context_decode_with_dumps(context, token, requests.data(), requests.size(), &Core::on_dump,
                                                         &Core::on_dump_logits, &job),
                      "decode with layer dumps");
    if (!status.ok() && !job.error.empty()) return {ErrorCode::kIo, job.error};
    return status;
  }

  Status embedding(const std::vector<TokenId> &tokens, const std::size_t layer, std::vector<float> *hidden) {
    auto status = ready(hidden);
    if (!status.ok()) return status;
    if (layer >= config.layers) return invalid("the embedding layer lies outside the model");
    const std::vector<LayerDump> dumps;  // block outputs come through the dump tap of that block
    std::vector<evo_b200_dump_request> requests{{layer, EVO_B200_DUMP_BLOCK_OUTPUT}};
    std::vector<std::uint8_t> bytes;
    for (const TokenId token : tokens) {
      if (token > 0xffU) return invalid("byte-level models take token ids below 256");
      bytes.push_back(static_cast<std::uint8_t>(token));
    }
    if (bytes.empty()) return invalid("an embedding needs at least one token");
    evo_batch *batch = nullptr;
    status = from_abi(evo_batch_create(1, &batch), "create a batch");
    if (!status.ok()) return status;
    status = from_abi(evo_batch_add_sequence(batch, bytes.data(), bytes.size()), "add the sequence");
    hidden->clear();
    std::vector<float> logits;
    struct Capture final {
      Rows hidden, logits;
    } capture{Rows{hidden}, Rows{&logits}};
    if (status.ok())
      status = from_abi(
          evo_b200_context_prefill_with_dumps(
              context, batch, requests.data(), requests.size(), 0,
              [](std::size_t, std::int32_t, const float *values, std::size_t rows, std::size_t columns, void *user) {
                return gather(values, rows, columns, 0, &static_cast<Capture *>(user)->hidden);
              },
              [](const float *values, std::size_t rows, std::size_t columns, std::size_t offset, void *user) {
                return gather(values, rows, columns, offset, &static_cast<Capture *>(user)->logits);
              },
              &capture),
          "prefill with a block-output capture");
    evo_batch_free(batch);
    return status;
  }

  Status chunk_embedding(const std::vector<TokenId> &tokens, const std::size_t layer, std::vector<float> *hidden) {
    auto status = ready(hidden);
    if (!status.ok()) return status;
    if (tokens.empty()) return invalid("an embedding needs at least one token");
    hidden->clear();
    Rows rows{hidden};
    return from_abi(evo_b200_context_embed_tokens(context, tokens.data(), tokens.size(), layer, 0, &Core::gather, &rows),
                    "embedding of a continuation chunk");
  }

  std::size_t position() const { return context == nullptr ? 0 : evo_context_position(context); }
  std::size_t activation_capacity() const { return context == nullptr ? 0 : evo_b200_context_activation_capacity(context); }
};

Status not_offered(const char *what) {
  return {ErrorCode::kUnsupported, std::string(what) + " is not offered through the C ABI of this build"};
}

}  // namespace

// ---- free functions -------------------------------------------------------------------------------

std::size_t backend_warmup_tokens(const RuntimeModelConfig &config, const std::size_t arena_capacity) noexcept {
  // upstream's policy: production 7B-family models run one 128-token prefill while loading
  constexpr std::size_t warmup = 128;
  const bool family = config.model_id.rfind("evo2_7b", 0) == 0;
  return !config.test_fixture && family && arena_capacity >= warmup ? warmup : 0;
}

Status validate_runtime_exact_support(const RuntimeModelConfig &config, const InferenceProfile profile) {
  if (config.test_fixture || !inference_profile_is_exact(profile)) return Status::Ok();
  return require_official_exact_support(config.model_id);
}

Status read_runtime_model_config(const ModelFile &model, const bool allow_test_fixture, RuntimeModelConfig *const config) {
  if (config == nullptr) return invalid("the configuration output is null");
  std::string path;
  auto status = path_of(model, &path);
  if (!status.ok()) return status;
  return read_config(path, allow_test_fixture, config);
}

// ---- SingleGpuModel ---------------------------------------------------------------------------------

struct SingleGpuModel::Impl final {
  Core core;
  int device{-1};
};

SingleGpuModel::SingleGpuModel() : impl_(std::make_unique<Impl>()) {}
SingleGpuModel::~SingleGpuModel() = default;
SingleGpuModel::SingleGpuModel(SingleGpuModel &&) noexcept = default;
SingleGpuModel &SingleGpuModel::operator=(SingleGpuModel &&) noexcept = default;

Status SingleGpuModel::load(const ModelFile &model, const int device, const std::size_t context_capacity,
                            const bool allow_test_fixture, const InferenceProfile profile) {
  auto fresh = std::make_unique<Impl>();
  auto status = fresh->core.load(model, {device}, context_capacity, allow_test_fixture, profile, 0);
  if (!status.ok()) return status;
  fresh->device = device;
  impl_ = std::move(fresh);
  return Status::Ok();
}

Status SingleGpuModel::prefill(const std::vector<TokenId> &tokens, std::vector<float> *logits,
                               const std::optional<LayerDump> &dump) {
  std::vector<LayerDump> dumps;
  if (dump.has_value()) dumps.push_back(*dump);
  return impl_->core.prefill_with_dumps(tokens, logits, dumps, false);
}
Status SingleGpuModel::prefill_with_dumps(const std::vector<TokenId> &tokens, std::vector<float> *logits,
                                          const std::vector<LayerDump> &dumps) {
  return impl_->core.prefill_with_dumps(tokens, logits, dumps, false);
}
Status SingleGpuModel::prefill_stateless(const std::vector<TokenId> &tokens, std::vector<float> *logits) {
  return impl_->core.prefill(tokens, EVO_B200_PREFILL_STATELESS, logits, "stateless prefill");
}
Status SingleGpuModel::prefill_cached(const std::vector<TokenId> &tokens, std::vector<float> *logits) {
  return impl_->core.prefill(tokens, EVO_B200_PREFILL_CACHED, logits, "cached prefill");
}
Status SingleGpuModel::prefill_cached_with_dumps(const std::vector<TokenId> &tokens, std::vector<float> *logits,
                                                 const std::vector<LayerDump> &dumps) {
  return impl_->core.prefill_with_dumps(tokens, logits, dumps, true);
}
Status SingleGpuModel::prefill_chunk(const std::vector<TokenId> &tokens, std::vector<float> *logits) {
  return impl_->core.prefill(tokens, EVO_B200_PREFILL_CHUNK, logits, "prefill chunk");
}
Status SingleGpuModel::prefill_embedding(const std::vector<TokenId> &tokens, const std::size_t layer,
                                         std::vector<float> *embedding) {
  return impl_->core.embedding(tokens, layer, embedding);
}
Status SingleGpuModel::prefill_chunk_embedding(const std::vector<TokenId> &tokens, const std::size_t layer,
                                               std::vector<float> *embedding) {
  return impl_->core.chunk_embedding(tokens, layer, embedding);
}
Status SingleGpuModel::decode(const TokenId token, std::vector<float> *logits) { return impl_->core.decode(token, logits); }
Status SingleGpuModel::decode_with_dumps(const TokenId token, std::vector<float> *logits,
                                         const std::vector<LayerDump> &dumps) {
  return impl_->core.decode_with_dumps(token, logits, dumps);
}
const RuntimeModelConfig &SingleGpuModel::config() const noexcept { return impl_->core.config; }
std::size_t SingleGpuModel::position() const noexcept { return impl_->core.position(); }
std::size_t SingleGpuModel::activation_capacity() const noexcept { return impl_->core.activation_capacity(); }
bool SingleGpuModel::uses_q8_kv_cache() const noexcept { return impl_->core.q8; }
int SingleGpuModel::device() const noexcept { return impl_->device; }

// ---- PipelineModel ----------------------------------------------------------------------------------

struct PipelineModel::Impl final {
  Core core;
};

PipelineModel::PipelineModel() : impl_(std::make_unique<Impl>()) {}
PipelineModel::~PipelineModel() = default;
PipelineModel::PipelineModel(PipelineModel &&) noexcept = default;
PipelineModel &PipelineModel::operator=(PipelineModel &&) noexcept = default;

Status PipelineModel::load(const ModelFile &model, const std::vector<int> &devices, const std::size_t context_capacity,
                           const bool allow_test_fixture, const InferenceProfile profile, const std::size_t layer_limit) {
  auto fresh = std::make_unique<Impl>();
  auto status = fresh->core.load(model, devices, context_capacity, allow_test_fixture, profile, layer_limit);
  if (!status.ok()) return status;
  impl_ = std::move(fresh);
  return Status::Ok();
}

Status PipelineModel::initialize_shared(const PipelineModel &source, const std::size_t context_capacity,
                                        const InferenceProfile profile) {
  if (source.impl_ == nullptr || source.impl_->core.weights == nullptr) return invalid("the source model is not loaded");
  auto status = validate_runtime_exact_support(source.impl_->core.config, profile);
  if (!status.ok()) return status;
  auto fresh = std::make_unique<Impl>();
  fresh->core.weights = source.impl_->core.weights;
  fresh->core.config = source.impl_->core.config;
  fresh->core.devices = source.impl_->core.devices;
  status = fresh->core.make_context(context_capacity, profile);
  if (!status.ok()) return status;
  impl_ = std::move(fresh);
  return Status::Ok();
}

Status PipelineModel::prefill(const std::vector<TokenId> &tokens, std::vector<float> *logits,
                              const std::optional<LayerDump> &dump) {
  std::vector<LayerDump> dumps;
  if (dump.has_value()) dumps.push_back(*dump);
  return impl_->core.prefill_with_dumps(tokens, logits, dumps, false);
}
Status PipelineModel::prefill_with_dumps(const std::vector<TokenId> &tokens, std::vector<float> *logits,
                                         const std::vector<LayerDump> &dumps) {
  return impl_->core.prefill_with_dumps(tokens, logits, dumps, false);
}
Status PipelineModel::prefill_stateless(const std::vector<TokenId> &tokens, std::vector<float> *logits) {
  return impl_->core.prefill(tokens, EVO_B200_PREFILL_STATELESS, logits, "stateless prefill");
}
Status PipelineModel::prefill_cached(const std::vector<TokenId> &tokens, std::vector<float> *logits) {
  return impl_->core.prefill(tokens, EVO_B200_PREFILL_CACHED, logits, "cached prefill");
}
Status PipelineModel::prefill_cached_with_dumps(const std::vector<TokenId> &tokens, std::vector<float> *logits,
                                                const std::vector<LayerDump> &dumps) {
  return impl_->core.prefill_with_dumps(tokens, logits, dumps, true);
}
Status PipelineModel::prefill_chunk(const std::vector<TokenId> &tokens, std::vector<float> *logits) {
  return impl_->core.prefill(tokens, EVO_B200_PREFILL_CHUNK, logits, "prefill chunk");
}
Status PipelineModel::prefill_embedding(const std::vector<TokenId> &tokens, const std::size_t layer,
                                        std::vector<float> *embedding) {
  return impl_->core.embedding(tokens, layer, embedding);
}
Status PipelineModel::prefill_chunk_embedding(const std::vector<TokenId> &tokens, const std::size_t layer,
                                              std::vector<float> *embedding) {
  return impl_->core.chunk_embedding(tokens, layer, embedding);
}
Status PipelineModel::decode(const TokenId token, std::vector<float> *logits) { return impl_->core.decode(token, logits); }
Status PipelineModel::decode_with_dumps(const TokenId token, std::vector<float> *logits,
                                        const std::vector<LayerDump> &dumps) {
  return impl_->core.decode_with_dumps(token, logits, dumps);
}
Status PipelineModel::prefill_prefix(const std::vector<TokenId> &, std::vector<float> *) {
  return not_offered("a truncated forward pass (prefill_prefix)");
}
Status PipelineModel::prefill_chunk_prefix(const std::vector<TokenId> &, std::vector<float> *) {
  return not_offered("a truncated forward pass (prefill_chunk_prefix)");
}
Status PipelineModel::decode_prefix(TokenId, std::vector<float> *) {
  return not_offered("a truncated forward pass (decode_prefix)");
}
const RuntimeModelConfig &PipelineModel::config() const noexcept { return impl_->core.config; }
const std::vector<StageAssignment> &PipelineModel::stages() const noexcept { return impl_->core.stages; }
void PipelineModel::refresh_cache_bytes() noexcept { impl_->core.refresh_stages(); }
std::size_t PipelineModel::position() const noexcept { return impl_->core.position(); }
std::size_t PipelineModel::activation_capacity() const noexcept { return impl_->core.activation_capacity(); }
bool PipelineModel::uses_q8_kv_cache() const noexcept { return impl_->core.q8; }
bool PipelineModel::shares_weights_with(const PipelineModel &other) const noexcept {
  return impl_ != nullptr && other.impl_ != nullptr && impl_->core.weights != nullptr &&
         impl_->core.weights == other.impl_->core.weights;
}

}  // namespace evo::cuda
