// Weight upload: validates the exact tensor set of an artifact against its
// metadata (upstream src/cuda/model.cu:874-1001), plans contiguous pipeline
// stages and copies every tensor into one device slab per stage.  Two load-time
// re-layouts: head-major Wqkv rows become projection-major (upstream
// src/cuda/model.cu:286-307 does the equivalent), and the MLP up-projections
// l1 / l2 are row-interleaved in blocks of 128 so one tensor-core GEMM can
// apply the gate in its epilogue.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <set>

#include <mutex>

#include "../common.cuh"
#include "../ops_internal.hpp"
#include "model.hpp"

namespace evob {
namespace {

constexpr std::size_t kAlign = 256;
std::size_t aligned(const std::size_t bytes) { return (bytes + kAlign - 1) / kAlign * kAlign; }

struct Expected {
  std::string name;
  TensorType type;
  std::vector<std::size_t> shape;
};

std::vector<Expected> expected_block_tensors(const ModelConfig &c, const std::size_t layer) {
  const std::string p = "blocks." + std::to_string(layer) + ".";
  const std::size_t D = c.width, I = c.inner_width;
  std::vector<Expected> list;
  list.push_back({p + "pre_norm.scale", TensorType::kF32, {D}});
  const MixerType type = c.mixers[layer];
  if (type == MixerType::kAttention) {
    list.push_back({p + "inner_mha_cls.out_proj.bias", TensorType::kBF16, {D}});
    list.push_back({p + "inner_mha_cls.out_proj.weight", TensorType::kBF16, {D, D}});
    list.push_back({p + "inner_mha_cls.Wqkv.weight", TensorType::kBF16, {3 * D, D}});
    list.push_back({p + "inner_mha_cls.rotary_emb.inv_freq", TensorType::kF32, {c.head_dim() / 2}});
  } else {
    list.push_back({p + "out_filter_dense.bias", TensorType::kBF16, {D}});
    list.push_back({p + "out_filter_dense.weight", TensorType::kBF16, {D, D}});
    if (c.fp8_projection) {
      list.push_back({p + "projections.fp8_runtime_scales", TensorType::kF32, {2}});
      list.push_back({p + "projections.weight", TensorType::kE4M3, {3 * D, D}});
    } else {
      list.push_back({p + "projections.weight", TensorType::kBF16, {3 * D, D}});
    }
    list.push_back({p + "filter.short_filter_weight", TensorType::kBF16, {3 * D, 1, c.short_taps}});
    if (type == MixerType::kHcs) {
      list.push_back({p + "filter.h", TensorType::kBF16, {c.hcs_groups, 1, c.hcs_taps}});
    } else if (type == MixerType::kHcm) {
      list.push_back({p + "filter.D", TensorType::kBF16, {D}});
      list.push_back({p + "filter.h", c.hcm_filter_f32 ? TensorType::kF32 : TensorType::kBF16,
                      {c.hcm_groups, 1, c.hcm_taps}});
    } else {
      list.push_back({p + "filter.D", TensorType::kBF16, {D}});
      list.push_back({p + "filter.log_poles", TensorType::kF32, {D, c.state_size, 1}});
      list.push_back({p + "filter.residues", TensorType::kF32, {D, c.state_size}});
    }
  }
  list.push_back({p + "mlp.l1.weight", TensorType::kBF16, {I, D}});
  list.push_back({p + "mlp.l2.weight", TensorType::kBF16, {I, D}});
  list.push_back({p + "mlp.l3.weight", TensorType::kBF16, {D, I}});
  list.push_back({p + "post_norm.scale", TensorType::kF32, {D}});
  return list;
}

int lookup(const ModelFile &file, const Expected &e, const TensorView **out) {
  const TensorView *tensor = file.find(e.name);
  if (tensor == nullptr) return fail(kModelFormat, "required tensor is missing: " + e.name);
  if (tensor->type != e.type || tensor->shape != e.shape)
    return fail(kModelFormat, "tensor has an unexpected dtype or shape: " + e.name);
  *out = tensor;
  return kOk;
}

bool gate_fusable(const ModelConfig &c) {
  return c.inner_width % 128 == 0 && c.width % 8 == 0 && c.width >= 64;
}

// Cursor over a stage slab.
struct Uploader {
  unsigned char *base = nullptr;
  std::size_t offset = 0;
  cudaStream_t stream = nullptr;
  bool dry_run = true;

  void *place(const std::size_t bytes) {
    void *p = dry_run ? nullptr : base + offset;
    offset += aligned(bytes);
    return p;
  }
  int copy(void *dst, const void *src, const std::size_t bytes) {
    if (dry_run || bytes == 0) return kOk;
    if (cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, stream) != cudaSuccess)
      return fail(kCuda, "weight upload failed");
    return kOk;
  }
  int tensor(const TensorView &t, const void **out) {
    void *dst = place(t.bytes);
    *out = dst;
    return copy(dst, t.data, t.bytes);
  }
};

int upload_layer(const ModelFile &file, const ModelConfig &c, const std::size_t layer,
                 Uploader *up, LayerWeights *w, std::vector<unsigned char> *host_scratch) {
  const std::vector<Expected> expected = expected_block_tensors(c, layer);
  std::vector<const TensorView *> t(expected.size());
  for (std::size_t i = 0; i < expected.size(); ++i) {
    const int status = lookup(file, expected[i], &t[i]);
    if (status != kOk) return status;
    w->payload_bytes += t[i]->bytes;
  }
  const auto by_suffix = [&](const char *suffix) -> const TensorView * {
    const std::string s(suffix);
    for (const TensorView *view : t)
      if (view->name.size() >= s.size() &&
          view->name.compare(view->name.size() - s.size(), s.size(), s) == 0)
        return view;
    return nullptr;
  };
  w->type = c.mixers[layer];
  const void *p = nullptr;
  int status = up->tensor(*by_suffix("pre_norm.scale"), &p);
  w->pre_norm = static_cast<const float *>(p);
  if (status == kOk) status = up->tensor(*by_suffix("post_norm.scale"), &p);
  w->post_norm = static_cast<const float *>(p);
  if (status != kOk) return status;
  if (w->type == MixerType::kAttention) {
    if ((status = up->tensor(*by_suffix("out_proj.bias"), &w->out_bias)) != kOk) return status;
    if ((status = up->tensor(*by_suffix("out_proj.weight"), &w->out_weight)) != kOk) return status;
    if ((status = up->tensor(*by_suffix("rotary_emb.inv_freq"), &p)) != kOk) return status;
    w->inverse_frequency = static_cast<const float *>(p);
    const TensorView &qkv = *by_suffix("Wqkv.weight");
    if (c.qkv_source_head_major && !up->dry_run) {
      // rows [head][q|k|v][dim] -> [q|k|v][head][dim]
      const std::size_t D = c.width, hd = c.head_dim(), row_bytes = D * 2;
      host_scratch->resize(qkv.bytes);
      for (std::size_t head = 0; head < c.heads; ++head)
        for (std::size_t part = 0; part < 3; ++part)
          std::memcpy(host_scratch->data() + (part * D + head * hd) * row_bytes,
                      qkv.data + (head * 3 * hd + part * hd) * row_bytes, hd * row_bytes);
      void *dst = up->place(qkv.bytes);
      w->projection = dst;
      if ((status = up->copy(dst, host_scratch->data(), qkv.bytes)) != kOk) return status;
      // the scratch buffer is reused by the next attention layer
      if (cudaStreamSynchronize(up->stream) != cudaSuccess) return fail(kCuda, "weight upload failed");
    } else {
      if ((status = up->tensor(qkv, &w->projection)) != kOk) return status;
    }
  } else {
    if ((status = up->tensor(*by_suffix("out_filter_dense.bias"), &w->out_bias)) != kOk) return status;
    if ((status = up->tensor(*by_suffix("out_filter_dense.weight"), &w->out_weight)) != kOk) return status;
    if ((status = up->tensor(*by_suffix("projections.weight"), &w->projection)) != kOk) return status;
    if (c.fp8_projection) {
      const TensorView &scales = *by_suffix("fp8_runtime_scales");
      float values[2];
      std::memcpy(values, scales.data, sizeof(values));
      if (!(values[0] > 0.0F) || !std::isfinite(values[0]) || !std::isfinite(values[1]))
        return fail(kModelFormat, "fp8_runtime_scales are invalid: " + scales.name);
      w->projection_input_scale = values[0];
      w->projection_output_scale = values[1];
    }
    if ((status = up->tensor(*by_suffix("short_filter_weight"), &w->short_filter)) != kOk) return status;
    if (w->type != MixerType::kHcl) {
      if ((status = up->tensor(*by_suffix("filter.h"), &w->inner_filter)) != kOk) return status;
    }
    if (w->type != MixerType::kHcs) {
      if ((status = up->tensor(*by_suffix("filter.D"), &w->direct)) != kOk) return status;
    }
    if (w->type == MixerType::kHcl) {
      if ((status = up->tensor(*by_suffix("filter.log_poles"), &p)) != kOk) return status;
      w->log_poles = static_cast<const float *>(p);
      if ((status = up->tensor(*by_suffix("filter.residues"), &p)) != kOk) return status;
      w->residues = static_cast<const float *>(p);
    }
  }
  const TensorView &l1 = *by_suffix("mlp.l1.weight"), &l2 = *by_suffix("mlp.l2.weight");
  if (gate_fusable(c)) {
    const std::size_t block_bytes = 128 * c.width * 2;
    unsigned char *dst = static_cast<unsigned char *>(up->place(l1.bytes + l2.bytes));
    w->l12 = dst;
    for (std::size_t block = 0; block < c.inner_width / 128 && !up->dry_run; ++block) {
      if ((status = up->copy(dst + (2 * block) * block_bytes, l1.data + block * block_bytes,
                             block_bytes)) != kOk)
        return status;
      if ((status = up->copy(dst + (2 * block + 1) * block_bytes, l2.data + block * block_bytes,
                             block_bytes)) != kOk)
        return status;
    }
  } else {
    if ((status = up->tensor(l1, &w->l1)) != kOk) return status;
    if ((status = up->tensor(l2, &w->l2)) != kOk) return status;
  }
  return up->tensor(*by_suffix("mlp.l3.weight"), &w->l3);
}

}  // namespace

StageWeights::~StageWeights() {
  if (slab != nullptr || ffn_slab != nullptr) {
    int previous = 0;
    cudaGetDevice(&previous);
    cudaSetDevice(device);
    if (slab != nullptr) cudaFree(slab);
    if (ffn_slab != nullptr) cudaFree(ffn_slab);
    cudaSetDevice(previous);
  }
}

// Per-tensor E4M3 copies of the output and MLP projection weights:
// code = E4M3(w * q), q = 448 / max|w| (the algebra of upstream's checkpoint
// converter for the Hyena input projections, tools/evo/checkpoint.py:100-112).
int StageWeights::ensure_fp8_ffn(const ModelConfig &c) {
  static std::mutex mutex;
  std::lock_guard<std::mutex> lock(mutex);
  if (ffn_slab != nullptr) return kOk;
  const std::size_t D = c.width, I = c.inner_width;
  for (const LayerWeights &w : layers)
    if (w.l12 == nullptr)
      return fail(kUnsupported, "the FP8 FFN profile needs the gate-fused MLP layout (inner width % 128 == 0)");
  if (D % 16 != 0 || I % 16 != 0) return fail(kUnsupported, "the FP8 FFN profile needs widths divisible by 16");
  int previous = 0;
  cudaGetDevice(&previous);
  struct Restore {
    int device;
    ~Restore() { cudaSetDevice(device); }
  } restore{previous};
  if (cudaSetDevice(device) != cudaSuccess) return fail(kCuda, "cannot select the stage's device");
  const std::size_t per_layer = aligned(D * D) + aligned(2 * I * D) + aligned(D * I);
  void *slab_memory = nullptr;
  if (cudaMalloc(&slab_memory, per_layer * layers.size() + 256) != cudaSuccess)
    return fail(kCuda, "cannot allocate " + std::to_string((per_layer * layers.size()) >> 20) +
                           " MiB for the FP8 FFN weights on device " + std::to_string(device));
  cudaStream_t stream = nullptr;
  unsigned int *amax_word = nullptr;
  int status = kOk;
  if (cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking) != cudaSuccess ||
      cudaMalloc(reinterpret_cast<void **>(&amax_word), sizeof(unsigned int)) != cudaSuccess)
    status = fail(kCuda, "cannot set up the FP8 FFN weight conversion");
  unsigned char *cursor = static_cast<unsigned char *>(slab_memory);
  const auto convert = [&](const void *source, const std::size_t elements, const void **codes, float *dequant) {
    if (status != kOk) return;
    status = amax_bf16(source, elements, amax_word, stream);
    unsigned int bits = 0;
    if (status == kOk && (cudaMemcpyAsync(&bits, amax_word, sizeof(bits), cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
                          cudaStreamSynchronize(stream) != cudaSuccess))
      status = fail(kCuda, "cannot read a weight's magnitude");
    if (status != kOk) return;
    bits = std::min(bits, 0x7f7fU) << 16U;
    float amax = 0.0F;
    std::memcpy(&amax, &bits, sizeof(amax));
    const float quant = amax > 0.0F ? 448.0F / amax : 1.0F;
    status = quantize_bf16(source, elements, quant, cursor, nullptr, stream);
    *codes = cursor;
    *dequant = 1.0F / quant;
    cursor += aligned(elements);
  };
  for (LayerWeights &w : layers) {
    convert(w.out_weight, D * D, &w.out_codes, &w.out_dequant);
    convert(w.l12, 2 * I * D, &w.l12_codes, &w.l12_dequant);
    convert(w.l3, D * I, &w.l3_codes, &w.l3_dequant);
  }
  if (status == kOk && cudaStreamSynchronize(stream) != cudaSuccess)
    status = fail(kCuda, "FP8 FFN weight conversion failed");
  if (amax_word != nullptr) cudaFree(amax_word);
  if (stream != nullptr) cudaStreamDestroy(stream);
  if (status != kOk) {
    cudaFree(slab_memory);
    for (LayerWeights &w : layers) w.out_codes = w.l12_codes = w.l3_codes = nullptr;
    return status;
  }
  ffn_slab = slab_memory;
  ffn_slab_bytes = per_layer * layers.size();
  return kOk;
}

int check_tensor_set(const ModelFile &file, const ModelConfig &c) {
  std::set<std::string> expected_names = {"embedding_layer.weight", "unembed.weight", "norm.scale"};
  const TensorView *view = nullptr;
  int status;
  if ((status = lookup(file, {"embedding_layer.weight", TensorType::kBF16, {c.vocab, c.width}}, &view)) != kOk ||
      (status = lookup(file, {"unembed.weight", TensorType::kBF16, {c.vocab, c.width}}, &view)) != kOk ||
      (status = lookup(file, {"norm.scale", TensorType::kF32, {c.width}}, &view)) != kOk)
    return status;
  for (std::size_t layer = 0; layer < c.layers; ++layer)
    for (const Expected &e : expected_block_tensors(c, layer)) {
      if ((status = lookup(file, e, &view)) != kOk) return status;
      expected_names.insert(e.name);
    }
  for (const TensorView &tensor : file.tensors())
    if (expected_names.count(tensor.name) == 0)
      return fail(kModelFormat, "unknown tensor for model profile '" + c.model_id + "': " + tensor.name);
  return kOk;
}

int load_weights(const ModelFile &file, const std::vector<int> &devices,
                 const bool allow_test_fixture, const std::size_t layer_limit,
                 std::shared_ptr<ModelWeights> *out, const std::size_t slice_index,
                 const std::size_t slice_count) {
  if (out == nullptr) return fail(kInvalidArgument, "model output is null");
  const bool sliced = slice_count > 1;
  if (slice_count == 0 || slice_count > 8 || slice_index >= slice_count ||
      (sliced && devices.size() != 1))
    return fail(kInvalidArgument, "a pipeline slice is one of 1..8 stages on exactly one device");
  if (devices.empty() || devices.size() > 8)
    return fail(kInvalidArgument, "the layer pipeline takes 1 to 8 CUDA devices");
  int device_count = 0;
  if (cudaGetDeviceCount(&device_count) != cudaSuccess || device_count == 0)
    return fail(kCuda, "no CUDA device is available");
  for (std::size_t i = 0; i < devices.size(); ++i) {
    if (devices[i] < 0 || devices[i] >= device_count)
      return fail(kInvalidArgument, "CUDA device index is out of range");
    for (std::size_t j = 0; j < i; ++j)
      if (devices[j] == devices[i])
        return fail(kInvalidArgument, "CUDA devices of a pipeline must be distinct");
  }
  auto weights = std::make_shared<ModelWeights>();
  int status = read_model_config(file, allow_test_fixture, &weights->config);
  if (status != kOk) return status;
  ModelConfig &c = weights->config;
  const std::size_t layers = layer_limit == 0 ? c.layers : layer_limit;
  const std::size_t stage_count = sliced ? slice_count : devices.size();
  if (layers > c.layers || layers < stage_count)
    return fail(kInvalidArgument, "CUDA layer limit must cover at least one layer per device");

  // exact tensor set
  std::set<std::string> expected_names = {"embedding_layer.weight", "unembed.weight", "norm.scale"};
  const TensorView *embedding = nullptr, *unembed = nullptr, *norm = nullptr;
  if ((status = lookup(file, {"embedding_layer.weight", TensorType::kBF16, {c.vocab, c.width}}, &embedding)) != kOk ||
      (status = lookup(file, {"unembed.weight", TensorType::kBF16, {c.vocab, c.width}}, &unembed)) != kOk ||
      (status = lookup(file, {"norm.scale", TensorType::kF32, {c.width}}, &norm)) != kOk)
    return status;
  std::vector<std::size_t> layer_bytes(layers, 0);
  for (std::size_t layer = 0; layer < c.layers; ++layer)
    for (const Expected &e : expected_block_tensors(c, layer)) {
      const TensorView *view = nullptr;
      if ((status = lookup(file, e, &view)) != kOk) return status;
      expected_names.insert(e.name);
      if (layer < layers) layer_bytes[layer] += view->bytes;
    }
  for (const TensorView &view : file.tensors())
    if (expected_names.count(view.name) == 0)
      return fail(kModelFormat, "unknown tensor for model profile '" + c.model_id + "': " + view.name);

  // Upstream's byte-balanced split serves its limit of four devices.  Beyond it a stage holds
  // only a few blocks, and a greedy byte target then leaves one stage a block more than its
  // neighbours (4/5/4/4/4/4/4/3 for 32 blocks on 8 devices) although every block costs about the
  // same time; the slowest stage sets the pipeline's rate, so equal block counts are used there.
  const auto plan = plan_stages(layer_bytes, stage_count, c.test_fixture || stage_count > 4);
  if (plan.size() != stage_count) return fail(kInternal, "stage planning failed");
  weights->slice_index = slice_index;
  weights->slice_count = slice_count;
  int previous_device = 0;
  cudaGetDevice(&previous_device);
  std::vector<unsigned char> host_scratch;
  for (std::size_t s = 0; s < stage_count && status == kOk; ++s) {
    if (sliced && s != slice_index) continue;
    auto stage = std::make_shared<StageWeights>();
    stage->device = sliced ? devices[0] : devices[s];
    // the tied head runs where the last block runs
    const bool holds_embedding = s == 0 || (sliced && s + 1 == stage_count);
    stage->layer_begin = plan[s].first;
    stage->layer_end = plan[s].second;
    stage->layers.resize(stage->layer_end - stage->layer_begin);
    for (int pass = 0; pass < 2 && status == kOk; ++pass) {
      Uploader up;
      up.dry_run = pass == 0;
      if (pass == 1) {
        if (cudaSetDevice(stage->device) != cudaSuccess ||
            cudaMalloc(&stage->slab, stage->slab_bytes) != cudaSuccess) {
          status = fail(kCuda, "cannot allocate " + std::to_string(stage->slab_bytes >> 20) +
                                   " MiB of weights on device " + std::to_string(stage->device));
          stage->slab = nullptr;
          break;
        }
        up.base = static_cast<unsigned char *>(stage->slab);
        if (cudaStreamCreateWithFlags(&up.stream, cudaStreamNonBlocking) != cudaSuccess) {
          status = fail(kCuda, "cannot create the upload stream");
          break;
        }
      }
      if (holds_embedding) {
        const void *p = nullptr;
        status = up.tensor(*embedding, &stage->embedding);
        if (status == kOk) status = up.tensor(*norm, &p);
        stage->final_norm = static_cast<const float *>(p);
      }
      for (std::size_t layer = stage->layer_begin; layer < stage->layer_end && status == kOk; ++layer) {
        LayerWeights scratch_weights;
        LayerWeights *target = pass == 1 ? &stage->layers[layer - stage->layer_begin] : &scratch_weights;
        status = upload_layer(file, c, layer, &up, target, &host_scratch);
      }
      if (pass == 0) {
        stage->slab_bytes = up.offset;
      } else if (up.stream != nullptr) {
        if (status == kOk && cudaStreamSynchronize(up.stream) != cudaSuccess)
          status = fail(kCuda, "weight upload failed");
        cudaStreamDestroy(up.stream);
      }
    }
    stage->weight_bytes = (holds_embedding ? embedding->bytes + unembed->bytes + norm->bytes : 0);
    for (const LayerWeights &w : stage->layers) stage->weight_bytes += w.payload_bytes;
    weights->stages.push_back(std::move(stage));
  }
  cudaSetDevice(previous_device);
  if (status != kOk) return status;
  *out = std::move(weights);
  return kOk;
}

}  // namespace evob
