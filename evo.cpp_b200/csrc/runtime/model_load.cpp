// Model configuration, stage planning and weight upload.
//
// read_model_config follows upstream's metadata contract
// (src/cuda/model.cu:517-870): typed config.* keys, semantic flags that must
// equal the supported Evo 2 profile, projection / medium-filter dtype keys,
// fixture permission.  One deliberate difference: a registered model id may
// carry E4M3 projections even where upstream's registry row is BF16 (e.g. a
// 7B-shaped FP8 artifact); the tensor set must still be exactly consistent
// with the metadata.
#include <algorithm>
#include <cmath>
#include <cstring>

#include "../common.cuh"
#include "../ops_internal.hpp"
#include "model.hpp"

namespace evob {
namespace {

struct KnownModel {
  const char *id;
  std::size_t width, layers, heads, inner, hcs_groups, hcm_groups;
};
// Shapes of the official Evo 2 family (upstream src/model_registry.cpp:50-100).
const KnownModel kKnownModels[] = {
    {"evo2_1b_base", 1920, 25, 15, 5120, 128, 128},
    {"evo2_7b", 4096, 32, 32, 11264, 256, 256},
    {"evo2_7b_base", 4096, 32, 32, 11008, 256, 256},
    {"evo2_7b_262k", 4096, 32, 32, 11008, 256, 256},
    {"evo2_20b", 8192, 24, 64, 22528, 512, 512},
    {"evo2_40b", 8192, 50, 64, 22528, 512, 512},
    {"evo2_40b_base", 8192, 50, 64, 21888, 512, 512},
    {"evo2_40b_bionemo_bf16", 8192, 50, 64, 22528, 512, 512},
};

#define EVOB_TRY(expr)              \
  do {                              \
    const int status__ = (expr);    \
    if (status__ != kOk) return status__; \
  } while (0)

}  // namespace

int read_model_config(const ModelFile &file, const bool allow_test_fixture,
                      ModelConfig *config) {
  if (config == nullptr) return fail(kInvalidArgument, "model config output is null");
  ModelConfig c;
  std::string abi;
  EVOB_TRY(file.get_string("evo2.profile", &c.artifact_profile));
  EVOB_TRY(file.get_string("runtime.abi", &abi));
  EVOB_TRY(file.get_string("model.architecture", &c.architecture));
  if (c.artifact_profile != "evo2-runtime-v1" || abi != "evo2-safetensors-v1")
    return fail(kUnsupported, "artifact is not an evo2-runtime-v1 Safetensors model");
  if (c.architecture == "StripedHyena2Test") {
    EVOB_TRY(file.get_bool("fixture.synthetic", &c.test_fixture));
    if (!c.test_fixture || !allow_test_fixture)
      return fail(kUnsupported, "synthetic model fixtures require explicit test permission");
  } else if (c.architecture != "StripedHyena2") {
    return fail(kUnsupported, "artifact is not a registered StripedHyena2 architecture");
  }
  if (file.metadata("model.id") != nullptr) EVOB_TRY(file.get_string("model.id", &c.model_id));
  if (file.metadata("model.name") != nullptr) EVOB_TRY(file.get_string("model.name", &c.model_name));
  EVOB_TRY(file.get_u64("config.vocab_size", &c.vocab));
  EVOB_TRY(file.get_u64("config.hidden_size", &c.width));
  EVOB_TRY(file.get_u64("config.num_layers", &c.layers));
  EVOB_TRY(file.get_u64("config.num_attention_heads", &c.heads));
  EVOB_TRY(file.get_u64("config.state_size", &c.state_size));
  EVOB_TRY(file.get_u64("config.inner_mlp_size", &c.inner_width));
  EVOB_TRY(file.get_u64("config.short_filter_length", &c.short_taps));
  EVOB_TRY(file.get_u64("config.hcs_filter_length", &c.hcs_taps));
  EVOB_TRY(file.get_u64("config.hcm_filter_length", &c.hcm_taps));
  EVOB_TRY(file.get_u64("config.hcs_filter_groups", &c.hcs_groups));
  EVOB_TRY(file.get_u64("config.hcm_filter_groups", &c.hcm_groups));
  double value = 0;
  EVOB_TRY(file.get_f64("config.eps", &value));
  c.epsilon = static_cast<float>(value);
  EVOB_TRY(file.get_f64("config.rotary_emb_scaling_factor", &value));
  c.rope_scale = static_cast<float>(value);
  bool column_split = false;
  if (!c.test_fixture) {
    std::size_t num_filters = 0, max_batch = 0, multiple = 0, proj_groups = 0, hcl_groups = 0;
    EVOB_TRY(file.get_u64("config.num_filters", &num_filters));
    EVOB_TRY(file.get_u64("config.max_batch_size", &max_batch));
    EVOB_TRY(file.get_u64("config.inner_size_multiple_of", &multiple));
    EVOB_TRY(file.get_u64("config.proj_groups", &proj_groups));
    EVOB_TRY(file.get_u64("config.hcl_filter_groups", &hcl_groups));
    EVOB_TRY(file.get_u64("config.max_seqlen", &c.max_seqlen));
    if (num_filters != c.width || max_batch != 1 || multiple != 128 || proj_groups != 1 ||
        hcl_groups != c.width)
      return fail(kUnsupported,
                  "model filter/batch/projection metadata is not an official Evo 2 profile");
    EVOB_TRY(file.get_f64("config.rotary_emb_base", &value));
    c.rope_base = static_cast<float>(value);
    EVOB_TRY(file.get_bool("config.column_split", &column_split));
  } else {
    c.max_seqlen = static_cast<std::size_t>(-1);
    if (file.metadata("config.column_split") != nullptr)
      EVOB_TRY(file.get_bool("config.column_split", &column_split));
  }
  bool tie = false, split_hyena = true, interleave = false, flip = true, fp8 = false;
  EVOB_TRY(file.get_bool("config.tie_embeddings", &tie));
  EVOB_TRY(file.get_bool("config.column_split_hyena", &split_hyena));
  EVOB_TRY(file.get_bool("config.interleave", &interleave));
  EVOB_TRY(file.get_bool("config.hyena_flip_x1x2", &flip));
  if (file.metadata("config.use_fp8_input_projections") != nullptr)
    EVOB_TRY(file.get_bool("config.use_fp8_input_projections", &fp8));
  else if (!c.test_fixture)
    return fail(kModelFormat, "required metadata is missing: config.use_fp8_input_projections");
  if (!tie || (!c.test_fixture && !column_split) || split_hyena || !interleave || flip)
    return fail(kUnsupported, "model semantic flags do not match supported Evo 2");
  c.qkv_source_head_major = column_split;
  if (!c.test_fixture) {
    bool short_bias = true, activations = false, final_norm = false, qkv_bias = true,
         mha_bias = false, hyena_bias = false;
    EVOB_TRY(file.get_bool("config.short_filter_bias", &short_bias));
    EVOB_TRY(file.get_bool("config.evo2_style_activations", &activations));
    EVOB_TRY(file.get_bool("config.final_norm", &final_norm));
    EVOB_TRY(file.get_bool("config.qkv_proj_bias", &qkv_bias));
    EVOB_TRY(file.get_bool("config.mha_out_proj_bias", &mha_bias));
    EVOB_TRY(file.get_bool("config.hyena_out_proj_bias", &hyena_bias));
    std::string tokenizer, prefill, activation;
    EVOB_TRY(file.get_string("config.tokenizer_type", &tokenizer));
    EVOB_TRY(file.get_string("config.prefill_style", &prefill));
    EVOB_TRY(file.get_string("config.mlp_activation", &activation));
    if (short_bias || !activations || !final_norm || qkv_bias || !mha_bias || !hyena_bias ||
        tokenizer != "CharLevelTokenizer" || prefill != "fft" || activation != "gelu")
      return fail(kUnsupported, "model semantic metadata is not an official Evo 2 profile");
  }
  std::string projection_dtype;
  if (file.metadata("hyena_projection_dtype") != nullptr)
    EVOB_TRY(file.get_string("hyena_projection_dtype", &projection_dtype));
  else if (c.test_fixture || fp8)
    projection_dtype = fp8 ? "E4M3_SW" : "BF16";
  else
    return fail(kModelFormat, "required metadata is missing: hyena_projection_dtype");
  if (projection_dtype != "BF16" && projection_dtype != "E4M3_SW")
    return fail(kUnsupported, "unsupported Hyena projection dtype: " + projection_dtype);
  c.fp8_projection = projection_dtype == "E4M3_SW";
  if (c.fp8_projection != fp8)
    return fail(kModelFormat,
                "hyena_projection_dtype disagrees with config.use_fp8_input_projections");
  std::string hcm_dtype = "BF16";
  if (file.metadata("hcm_filter_dtype") != nullptr)
    EVOB_TRY(file.get_string("hcm_filter_dtype", &hcm_dtype));
  else if (!c.model_id.empty())
    return fail(kModelFormat, "registered models require hcm_filter_dtype metadata");
  if (hcm_dtype != "BF16" && hcm_dtype != "F32")
    return fail(kUnsupported, "unsupported medium-Hyena filter dtype: " + hcm_dtype);
  c.hcm_filter_f32 = hcm_dtype == "F32";
  if (!c.test_fixture && c.fp8_projection) {
    std::string reference;
    EVOB_TRY(file.get_string("fp8.reference", &reference));
    if (reference != "TransformerEngine-2.3-HYBRID")
      return fail(kUnsupported, "unsupported software-FP8 checkpoint reference: " + reference);
  } else if (!c.fp8_projection && file.metadata("fp8.reference") != nullptr) {
    return fail(kModelFormat, "BF16 Hyena projections must not declare fp8.reference");
  }
  std::vector<std::size_t> hcs, hcm, hcl, attention;
  EVOB_TRY(file.get_list("config.hcs_layer_idxs", &hcs));
  EVOB_TRY(file.get_list("config.hcm_layer_idxs", &hcm));
  EVOB_TRY(file.get_list("config.hcl_layer_idxs", &hcl));
  EVOB_TRY(file.get_list("config.attn_layer_idxs", &attention));
  if (c.vocab == 0 || c.width == 0 || c.heads == 0 || c.layers == 0 || c.width % c.heads != 0 ||
      c.head_dim() % 2 != 0 || c.head_dim() > 256 || c.state_size == 0 || c.state_size > 16 ||
      c.inner_width == 0 || c.short_taps != 3 || c.hcs_taps < 2 || c.hcm_taps < 2 ||
      c.hcs_taps > 128 || c.hcm_taps > 128 || c.hcs_groups == 0 || c.width % c.hcs_groups != 0 ||
      c.hcm_groups == 0 || c.width % c.hcm_groups != 0 || c.width % 2 != 0 ||
      !std::isfinite(c.epsilon) || c.epsilon <= 0.0F || !std::isfinite(c.rope_scale) ||
      c.rope_scale <= 0.0F)
    return fail(kUnsupported, "model dimensions are unsupported");
  c.mixers.assign(c.layers, MixerType::kHcs);
  std::vector<int> assigned(c.layers, 0);
  const auto mark = [&](const std::vector<std::size_t> &list, const MixerType type) {
    for (const std::size_t layer : list) {
      if (layer >= c.layers) return false;
      c.mixers[layer] = type;
      ++assigned[layer];
    }
    return true;
  };
  if (!mark(hcs, MixerType::kHcs) || !mark(hcm, MixerType::kHcm) || !mark(hcl, MixerType::kHcl) ||
      !mark(attention, MixerType::kAttention) ||
      std::any_of(assigned.begin(), assigned.end(), [](const int n) { return n != 1; }))
    return fail(kModelFormat, "layer index lists do not partition the blocks");
  if (!c.test_fixture) {
    if (c.model_id.empty()) return fail(kModelFormat, "required metadata is missing: model.id");
    const KnownModel *known = nullptr;
    for (const KnownModel &m : kKnownModels)
      if (c.model_id == m.id) known = &m;
    if (known == nullptr || known->width != c.width || known->layers != c.layers ||
        known->heads != c.heads || known->inner != c.inner_width ||
        known->hcs_groups != c.hcs_groups || known->hcm_groups != c.hcm_groups || c.vocab != 512)
      return fail(kUnsupported, "model metadata does not match a registered Evo 2 shape");
  }
  *config = std::move(c);
  return kOk;
}

std::vector<std::pair<std::size_t, std::size_t>> plan_stages(
    const std::vector<std::size_t> &layer_bytes, const std::size_t stage_count,
    const bool even_split) {
  std::vector<std::pair<std::size_t, std::size_t>> plan;
  const std::size_t layers = layer_bytes.size();
  if (stage_count == 0 || layers < stage_count) return plan;
  std::size_t begin = 0;
  if (even_split) {
    for (std::size_t s = 0; s < stage_count; ++s) {
      const std::size_t count = layers / stage_count + (s < layers % stage_count ? 1 : 0);
      plan.emplace_back(begin, begin + count);
      begin += count;
    }
    return plan;
  }
  std::size_t remaining = 0;
  for (const std::size_t b : layer_bytes) remaining += b;
  for (std::size_t s = 0; s < stage_count; ++s) {
    const std::size_t stages_left = stage_count - s;
    if (stages_left == 1) {
      plan.emplace_back(begin, layers);
      break;
    }
    const std::size_t target = (remaining + stages_left - 1) / stages_left;
    const std::size_t latest_end = layers - (stages_left - 1);
    std::size_t end = begin, assigned = 0;
    while (end < latest_end && (end == begin || assigned < target)) assigned += layer_bytes[end++];
    plan.emplace_back(begin, end);
    remaining -= assigned;
    begin = end;
  }
  return plan;
}

}  // namespace evob
