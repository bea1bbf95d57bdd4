// Per-context state and the block graph of the StripedHyena2 forward pass
// (upstream src/cuda/model.cu:1327-1944 run_mixer / run_blocks / forward and
// 2148-2366 PipelineModel).  One Stage per GPU owns a stream, an activation
// arena and the causal state of its blocks (FIR histories, modal state, KV
// cache).  Stages are chained with stream-ordered peer copies: no host
// synchronisation between stages, only the final logits read-back blocks.
#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "../common.cuh"
#include "../ops_internal.hpp"
#include "model.hpp"

namespace evob {

namespace {
constexpr std::size_t kArenaRows = 8192;       // upstream src/cuda/model.cu:31
constexpr std::size_t kFixtureArenaRows = 8;   // upstream src/cuda/model.cu:32

#define EVOB_TRY(expr)                    \
  do {                                    \
    const int status__ = (expr);          \
    if (status__ != kOk) return status__; \
  } while (0)

// Runs one operator launch; when the stage is profiling, brackets it with CUDA
// events on the stage stream and files the elapsed time under `category`.
#define EVOB_OP(category, expr)           \
  do {                                    \
    s.begin_op(category);                 \
    const int status__ = (expr);          \
    s.end_op();                           \
    if (status__ != kOk) return status__; \
  } while (0)

struct DeviceGuard {
  int previous = 0;
  explicit DeviceGuard(const int device) {
    cudaGetDevice(&previous);
    cudaSetDevice(device);
  }
  ~DeviceGuard() { cudaSetDevice(previous); }
};
}  // namespace

// Rows of history kept in front of a continuation chunk inside the activation
// buffers (>= the longest filter's reach of 127 + 2 featurizer rows, and a
// multiple of 16 so the tensor-core FIR tiles keep their alignment).
constexpr std::size_t kHistoryPad = 144;
constexpr std::size_t kSplitWorkspaceBytes = std::size_t{64} << 20;
constexpr std::size_t kQ8PageTokens = 16384;  // upstream src/cuda/model.cu:33

struct LayerState {
  float *short_cache = nullptr;  // [3D, short_taps-1]
  float *inner_cache = nullptr;  // [D, taps-1]
  float *modal_state = nullptr;  // [D, S]
  void *key_cache = nullptr, *value_cache = nullptr;  // [context, D] BF16
  // Pipelines only: the last projection rows of the previous wavefront chunk
  // ([history_rows, 3D] BF16).  The projection arena is shared by all blocks of
  // a stage, so a block's own history is parked here between chunks.
  void *history = nullptr;
  std::size_t history_rows = 0;
  // fast-q8-kv: page p holds positions [p * kQ8PageTokens, ...); pointers are mirrored in four
  // device arrays (key codes, value codes, key scales, value scales) that the kernels index
  std::vector<void *> q8_pages[4];
  void **q8_tables = nullptr;  // [4][page_count] device
  std::size_t q8_page_count = 0;
  Q8PageTable q8_table() const {
    Q8PageTable t;
    t.key = reinterpret_cast<std::int8_t *const *>(q8_tables);
    t.value = reinterpret_cast<std::int8_t *const *>(q8_tables + q8_page_count);
    t.key_scale = reinterpret_cast<float *const *>(q8_tables + 2 * q8_page_count);
    t.value_scale = reinterpret_cast<float *const *>(q8_tables + 3 * q8_page_count);
    t.page_tokens = kQ8PageTokens;
    return t;
  }
};

struct Context::Stage {
  std::shared_ptr<StageWeights> weights;
  int device = 0;
  cudaStream_t stream = nullptr;
  cudaEvent_t done = nullptr;
  std::vector<void *> allocations;
  std::size_t arena_bytes = 0, cache_bytes = 0;
  // activations
  void *hidden = nullptr, *residual = nullptr, *normalized = nullptr, *mixer_out = nullptr;
  void *codes = nullptr, *projection = nullptr, *query = nullptr, *gated = nullptr;
  void *codes_wide = nullptr;   // [T, I] E4M3 codes of the gated MLP activations (FP8 FFN profile)
  float *row_scale = nullptr;   // [T] dequantisation factor of the row-quantised operand in flight
  void *mlp_first = nullptr, *mlp_second = nullptr;
  void *short_filtered = nullptr, *x2 = nullptr, *x1 = nullptr, *value = nullptr, *pregate = nullptr;
  float *modal_scratch = nullptr;
  void *split_workspace = nullptr;  // F32 partial sums of split-K projections (<= 128 rows)
  // fast-q8-kv: BF16 images [context, D] of the keys and values one attention block at a time
  void *kv_image_key = nullptr, *kv_image_value = nullptr;
  std::uint32_t *tokens = nullptr;
  void *logits = nullptr;
  std::vector<LayerState> layers;

  // ---- optional per-operator timing
  bool profiling = false;
  std::vector<cudaEvent_t> events;    // pairs: start, stop
  std::vector<int> event_category;    // one per pair in use
  double category_ms[kProfileCategories] = {};
  std::uint64_t category_launches[kProfileCategories] = {};

  void begin_op(const int category) {
    if (!profiling) return;
    const std::size_t pair = event_category.size();
    while (events.size() < 2 * (pair + 1)) {
      cudaEvent_t event = nullptr;
      cudaEventCreate(&event);
      events.push_back(event);
    }
    event_category.push_back(category);
    cudaEventRecord(events[2 * pair], stream);
  }
  void end_op() {
    if (!profiling || event_category.empty()) return;
    cudaEventRecord(events[2 * (event_category.size() - 1) + 1], stream);
  }
  // Call after the stream has been synchronised.
  void collect_profile() {
    for (std::size_t pair = 0; pair < event_category.size(); ++pair) {
      float ms = 0.0F;
      if (cudaEventElapsedTime(&ms, events[2 * pair], events[2 * pair + 1]) == cudaSuccess) {
        category_ms[event_category[pair]] += ms;
        ++category_launches[event_category[pair]];
      }
    }
    event_category.clear();
  }

  // Advances (or rewinds) every row-indexed activation pointer by `rows`.
  void shift_rows(const long rows, const std::size_t D, const std::size_t I) {
    const auto move = [rows](void *&pointer, const std::size_t row_bytes) {
      if (pointer != nullptr)
        pointer = static_cast<unsigned char *>(pointer) + rows * static_cast<long>(row_bytes);
    };
    for (void **p : {&hidden, &residual, &normalized, &mixer_out, &query, &x2, &x1, &value, &pregate})
      move(*p, D * 2);
    move(codes, D);
    move(codes_wide, I);
    if (row_scale != nullptr) row_scale += rows;
    move(projection, D * 6);
    move(short_filtered, D * 6);
    for (void **p : {&gated, &mlp_first, &mlp_second}) move(*p, I * 2);
  }

  // Pages of one attention block up to position `tokens_end` (exclusive); new pointers are
  // written into the device tables in stream order.
  int ensure_q8_pages(LayerState &state, const std::size_t tokens_end, const std::size_t heads,
                      const std::size_t head_dim) {
    const std::size_t needed = (tokens_end + kQ8PageTokens - 1) / kQ8PageTokens;
    if (needed > state.q8_page_count) return fail(kInvalidArgument, "quantised KV cache capacity exceeded");
    for (std::size_t page = state.q8_pages[0].size(); page < needed; ++page) {
      for (int which = 0; which < 4; ++which) {
        void *memory = nullptr;
        const std::size_t bytes = which < 2 ? kQ8PageTokens * heads * head_dim : kQ8PageTokens * heads * sizeof(float);
        const int status = allocate(&memory, bytes, &cache_bytes);
        if (status != kOk) return status;
        state.q8_pages[which].push_back(memory);
        if (cudaMemcpyAsync(state.q8_tables + which * state.q8_page_count + page, &state.q8_pages[which][page],
                            sizeof(void *), cudaMemcpyHostToDevice, stream) != cudaSuccess)
          return fail(kCuda, "cannot publish a quantised KV page");
      }
    }
    return kOk;
  }

  int allocate(void **out, const std::size_t bytes, std::size_t *counter) {
    if (cudaMalloc(out, bytes == 0 ? 16 : bytes) != cudaSuccess)
      return fail(kCuda, "cannot allocate " + std::to_string(bytes >> 20) + " MiB on device " +
                             std::to_string(device));
    allocations.push_back(*out);
    *counter += bytes;
    return kOk;
  }
  ~Stage() {
    DeviceGuard guard(device);
    if (stream != nullptr) cudaStreamSynchronize(stream);
    for (void *p : allocations) cudaFree(p);
    for (cudaEvent_t event : events) cudaEventDestroy(event);
    if (done != nullptr) cudaEventDestroy(done);
    if (stream != nullptr) cudaStreamDestroy(stream);
  }
};

// ---- activation taps (upstream dump_matching & friends, src/cuda/model.cu:1583-1742)
namespace {

struct ScopedDeviceBuffer {
  void *data = nullptr;
  int reserve(const std::size_t bytes) {
    if (cudaMalloc(&data, bytes == 0 ? 16 : bytes) != cudaSuccess) {
      data = nullptr;
      return fail(kCuda, "cannot allocate " + std::to_string(bytes >> 20) + " MiB of dump scratch");
    }
    return kOk;
  }
  ~ScopedDeviceBuffer() {
    if (data != nullptr) cudaFree(data);
  }
};

// Hands `values` to every request of the plan that names (layer, point).
int deliver(const DumpPlan &plan, const std::size_t layer, const DumpPoint point,
            const std::vector<float> &values, const std::size_t rows, const std::size_t columns) {
  for (const DumpPlan::Request &request : plan.requests) {
    if (request.layer != layer || request.point != point) continue;
    const int status = plan.sink ? plan.sink(request, values.data(), rows, columns) : kOk;
    if (status != kOk) return fail(status, "dump consumer aborted the forward pass");
  }
  return kOk;
}

// BF16 [rows, columns] on the device -> F32 on the host -> sink.
int emit_bf16(cudaStream_t stream, const DumpPlan &plan, const std::size_t layer, const DumpPoint point,
              const void *device, const std::size_t rows, const std::size_t columns) {
  if (!plan.wants(layer, point)) return kOk;
  std::vector<std::uint16_t> raw(rows * columns);
  if (cudaMemcpyAsync(raw.data(), device, raw.size() * 2, cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
      cudaStreamSynchronize(stream) != cudaSuccess)
    return fail(kCuda, std::string("dump read-back failed: ") + cudaGetErrorString(cudaGetLastError()));
  std::vector<float> values(raw.size());
  for (std::size_t j = 0; j < raw.size(); ++j) {
    const std::uint32_t bits = static_cast<std::uint32_t>(raw[j]) << 16U;
    std::memcpy(&values[j], &bits, 4);
  }
  return deliver(plan, layer, point, values, rows, columns);
}

// F32 [rows, columns] on the device; only the last `active` columns of each row
// are reported (FIR histories are left-padded with zeros until they fill).
int emit_f32(cudaStream_t stream, const DumpPlan &plan, const std::size_t layer, const DumpPoint point,
             const float *device, const std::size_t rows, const std::size_t columns, const std::size_t active) {
  if (!plan.wants(layer, point)) return kOk;
  if (active > columns) return fail(kInternal, "active FIR cache columns exceed cache capacity");
  std::vector<float> padded(rows * columns);
  if (cudaMemcpyAsync(padded.data(), device, padded.size() * 4, cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
      cudaStreamSynchronize(stream) != cudaSuccess)
    return fail(kCuda, std::string("dump read-back failed: ") + cudaGetErrorString(cudaGetLastError()));
  if (active == columns) return deliver(plan, layer, point, padded, rows, columns);
  std::vector<float> values(rows * active);
  for (std::size_t row = 0; row < rows; ++row)
    std::copy_n(padded.begin() + static_cast<std::ptrdiff_t>(row * columns + columns - active), active,
                values.begin() + static_cast<std::ptrdiff_t>(row * active));
  return deliver(plan, layer, point, values, rows, active);
}

}  // namespace

const char *dump_point_name(const int point) {
  static const char *const names[static_cast<int>(DumpPoint::kDumpPoints)] = {
      "block_output", "pre_norm", "mixer_input_projection", "mixer_short_filter", "mixer_short_state",
      "mixer_inner_state", "mixer_x2", "mixer_x1", "mixer_value", "mixer_pregate", "mixer_state",
      "mixer_filter", "mixer_convolution", "mixer_output", "mixer_projection", "mixer_residual",
      "post_norm", "mlp_l1", "mlp_l2", "mlp_activation", "mlp_gated", "mlp_output"};
  return point >= 0 && point < static_cast<int>(DumpPoint::kDumpPoints) ? names[point] : "";
}

// Taps inside a Hyena mixer.  After an initial prefill the fused kernels have
// kept the featurizer output, the split and the pre-gate in registers, so they
// are recomputed here with the unfused operators (same roundings: the fused
// short-explicit operator is bit-identical to this sequence); after a
// continuation or decode step the unfused path has just left them in the arena.
int Context::dump_mixer_taps(Stage &s, const std::size_t i, const std::size_t rows, const Mode mode,
                             const DumpPlan &plan) {
  const ModelConfig &c = weights_->config;
  const LayerWeights &w = s.weights->layers[i];
  LayerState &state = s.layers[i];
  const std::size_t D = c.width, layer = s.weights->layer_begin + i;
  const bool initial = mode == Mode::kPrefill || mode == Mode::kStateless || mode == Mode::kCachedPrefill;
  const bool stateless = mode == Mode::kStateless;
  cudaStream_t stream = s.stream;
  if (initial) {
    EVOB_TRY(fir_prefill(s.projection, w.short_filter, false, nullptr, false, rows, 3 * D, 3 * D, c.short_taps,
                         true, s.short_filtered, nullptr, stream));
    EVOB_TRY(split_triples(s.short_filtered, rows, D, s.x2, s.x1, s.value, stream));
    EVOB_TRY(gate(s.x1, s.value, s.pregate, rows * D, false, stream));
  }
  const std::size_t seen = (initial ? 0 : position_) + rows;
  EVOB_TRY(emit_bf16(stream, plan, layer, DumpPoint::kMixerShortFilter, s.short_filtered, rows, 3 * D));
  if (!stateless)
    EVOB_TRY(emit_f32(stream, plan, layer, DumpPoint::kMixerShortState, state.short_cache, 3 * D,
                      c.short_taps - 1, std::min(seen, c.short_taps - 1)));
  EVOB_TRY(emit_bf16(stream, plan, layer, DumpPoint::kMixerX2, s.x2, rows, D));
  EVOB_TRY(emit_bf16(stream, plan, layer, DumpPoint::kMixerX1, s.x1, rows, D));
  EVOB_TRY(emit_bf16(stream, plan, layer, DumpPoint::kMixerValue, s.value, rows, D));
  if (w.type != MixerType::kHcl && !stateless) {
    const std::size_t taps = w.type == MixerType::kHcs ? c.hcs_taps : c.hcm_taps;
    EVOB_TRY(emit_f32(stream, plan, layer, DumpPoint::kMixerInnerState, state.inner_cache, D, taps - 1,
                      std::min(seen, taps - 1)));
  }
  if (w.type == MixerType::kHcl && !stateless)
    EVOB_TRY(emit_f32(stream, plan, layer, DumpPoint::kMixerState, state.modal_state, D, c.state_size,
                      c.state_size));
  EVOB_TRY(emit_bf16(stream, plan, layer, DumpPoint::kMixerPregate, s.pregate, rows, D));
  if (w.type == MixerType::kHcl && initial) {
    const bool filter = plan.wants(layer, DumpPoint::kMixerFilter);
    const bool convolution = plan.wants(layer, DumpPoint::kMixerConvolution);
    if (filter || convolution) {
      ScopedDeviceBuffer filter_values, convolution_values;
      if (filter) EVOB_TRY(filter_values.reserve(rows * D * 4));
      if (convolution) EVOB_TRY(convolution_values.reserve(rows * D * 4));
      EVOB_TRY(modal_taps(s.pregate, w.log_poles, w.residues, rows, D, c.state_size,
                          static_cast<float *>(filter_values.data), static_cast<float *>(convolution_values.data),
                          stream));
      if (filter)
        EVOB_TRY(emit_f32(stream, plan, layer, DumpPoint::kMixerFilter, static_cast<float *>(filter_values.data),
                          rows, D, D));
      if (convolution)
        EVOB_TRY(emit_f32(stream, plan, layer, DumpPoint::kMixerConvolution,
                          static_cast<float *>(convolution_values.data), rows, D, D));
    }
  }
  return kOk;
}

// Taps inside the MLP that the gate-fused up-projection never writes: l1(x),
// l2(x) and, in block 0, gelu(l1(x)).  The interleaved weight is multiplied
// once more without the gate; its output row is [l1 block 0 | l2 block 0 | l1
// block 1 | ...] in 128-column blocks, which two strided copies separate.
int Context::dump_mlp_taps(Stage &s, const std::size_t i, const std::size_t rows, const bool ffn8,
                           const DumpPlan &plan) {
  const ModelConfig &c = weights_->config;
  const LayerWeights &w = s.weights->layers[i];
  const std::size_t D = c.width, I = c.inner_width, layer = s.weights->layer_begin + i;
  const bool activation = layer == 0 && plan.wants(layer, DumpPoint::kMlpActivation);
  if (!plan.wants(layer, DumpPoint::kMlpL1) && !plan.wants(layer, DumpPoint::kMlpL2) && !activation) return kOk;
  cudaStream_t stream = s.stream;
  ScopedDeviceBuffer raw, first, second, activated;
  const void *l1_values = s.mlp_first, *l2_values = s.mlp_second;
  if (w.l12 != nullptr) {
    EVOB_TRY(raw.reserve(rows * 2 * I * 2));
    EVOB_TRY(first.reserve(rows * I * 2));
    EVOB_TRY(second.reserve(rows * I * 2));
    LinearArgs a;
    a.split_workspace = s.split_workspace;
    a.split_workspace_bytes = kSplitWorkspaceBytes;
    a.input = s.normalized;
    a.weight = w.l12;
    a.output = raw.data;
    a.rows = rows;
    a.in_features = D;
    a.out_features = 2 * I;
    if (ffn8) {  // the row-quantised operand of the gated product is still in s.codes
      a.input = s.codes;
      a.weight = w.l12_codes;
      a.operand_type = OperandType::kE4m3;
      a.alpha = w.l12_dequant;
      a.row_scale = s.row_scale;
    }
    EVOB_TRY(linear(a, stream));
    const std::size_t blocks = rows * (I / 128);
    if (cudaMemcpy2DAsync(first.data, 256, raw.data, 512, 256, blocks, cudaMemcpyDeviceToDevice, stream) !=
            cudaSuccess ||
        cudaMemcpy2DAsync(second.data, 256, static_cast<unsigned char *>(raw.data) + 256, 512, 256, blocks,
                          cudaMemcpyDeviceToDevice, stream) != cudaSuccess)
      return fail(kCuda, "dump de-interleave failed");
    l1_values = first.data;
    l2_values = second.data;
  }
  EVOB_TRY(emit_bf16(stream, plan, layer, DumpPoint::kMlpL1, l1_values, rows, I));
  EVOB_TRY(emit_bf16(stream, plan, layer, DumpPoint::kMlpL2, l2_values, rows, I));
  if (activation) {
    EVOB_TRY(activated.reserve(rows * I * 2));
    EVOB_TRY(gelu(l1_values, activated.data, rows * I, stream));
    EVOB_TRY(emit_bf16(stream, plan, layer, DumpPoint::kMlpActivation, activated.data, rows, I));
  }
  return kOk;
}

Context::~Context() {
  if (decode_graph_ != nullptr) cudaGraphExecDestroy(static_cast<cudaGraphExec_t>(decode_graph_));
}

// One decode step as a replayed CUDA graph.  The step's launches depend on the
// position only through the RoPE angle / KV append index and the number of
// cached keys, which the small-row attention kernels read from device memory,
// and through the FIR history counts, which are constant once the history is
// full; everything else is fixed addresses.  Returns kOk with *launched = false
// when the step has to take the ordinary path.
int Context::decode_step_graph(const std::uint32_t *host_token, bool *launched) {
  *launched = false;
  const ModelConfig &c = weights_->config;
  Stage &first = *stages_.front();
  DeviceGuard guard(first.device);
  cudaStream_t stream = first.stream;
  decode_position_host_ = static_cast<int>(position_);
  if (cudaMemcpyAsync(first.tokens, host_token, 4, cudaMemcpyHostToDevice, stream) != cudaSuccess ||
      cudaMemcpyAsync(device_position_, &decode_position_host_, 4, cudaMemcpyHostToDevice, stream) != cudaSuccess)
    return fail(kCuda, "token upload failed");
  if (decode_graph_ == nullptr) {
    if (cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
      cudaGetLastError();
      decode_graph_allowed_ = false;
      return kOk;
    }
    dynamic_position_ = device_position_;
    int status = embedding(first.tokens, first.weights->embedding, 1, c.width, c.vocab, first.hidden, stream);
    if (status == kOk) status = run_stage(first, 1, Mode::kDecode, -1, nullptr);
    if (status == kOk)
      status = rms_norm(first.hidden, first.weights->final_norm, 1, c.width, c.epsilon, first.normalized,
                        nullptr, 1.0F, stream);
    if (status == kOk) {
      LinearArgs a;
      a.split_workspace = first.split_workspace;
      a.split_workspace_bytes = kSplitWorkspaceBytes;
      a.dependent_launch = decode_dependent_launch_ && true;
      a.input = first.normalized;
      a.weight = first.weights->embedding;  // tied head
      a.output = first.logits;
      a.rows = 1;
      a.in_features = c.width;
      a.out_features = c.vocab;
      status = linear(a, stream);
    }
    dynamic_position_ = nullptr;
    cudaGraph_t graph = nullptr;
    const cudaError_t ended = cudaStreamEndCapture(stream, &graph);
    cudaGraphExec_t executable = nullptr;
    if (status != kOk || ended != cudaSuccess || graph == nullptr ||
        cudaGraphInstantiate(&executable, graph, 0) != cudaSuccess) {
      // nothing ran: the step falls back to ordinary launches, for good
      cudaGetLastError();
      if (graph != nullptr) cudaGraphDestroy(graph);
      decode_graph_allowed_ = false;
      return kOk;
    }
    cudaGraphDestroy(graph);
    decode_graph_ = executable;
  }
  if (cudaGraphLaunch(static_cast<cudaGraphExec_t>(decode_graph_), stream) != cudaSuccess)
    return fail(kCuda, std::string("decode graph launch failed: ") + cudaGetErrorString(cudaGetLastError()));
  *launched = true;
  return kOk;
}

int Context::create(std::shared_ptr<ModelWeights> weights, const std::size_t context_size,
                    const ExecutionProfile profile, const bool full_arena_for_fixtures,
                    std::unique_ptr<Context> *out, const bool q8_kv) {
  if (weights == nullptr || out == nullptr || context_size == 0)
    return fail(kInvalidArgument, "context arguments are invalid");
  const ModelConfig &c = weights->config;
  if (!c.test_fixture && context_size > c.max_seqlen)
    return fail(kInvalidArgument, "requested context exceeds model maximum of " +
                                      std::to_string(c.max_seqlen));
  std::unique_ptr<Context> context(new Context());
  context->weights_ = weights;
  context->profile_ = profile;
  context->q8_kv_ = q8_kv;
  if (const char *const parts = std::getenv("EVO_B200_FP8_FFN_PARTS"))
    context->fp8_ffn_parts_ = static_cast<unsigned>(std::strtoul(parts, nullptr, 0)) & 7U;
  context->context_size_ = context_size;
  context->arena_rows_ = std::min(
      context_size, c.test_fixture && !full_arena_for_fixtures ? kFixtureArenaRows : kArenaRows);
  const std::size_t T = context->arena_rows_ + kHistoryPad, D = c.width, I = c.inner_width;
  const bool fused_gate = !weights->stages.empty() && !weights->stages[0]->layers.empty() &&
                          weights->stages[0]->layers[0].l12 != nullptr;
  for (const auto &stage_weights : weights->stages) {
    auto stage = std::make_unique<Stage>();
    stage->weights = stage_weights;
    stage->device = stage_weights->device;
    DeviceGuard guard(stage->device);
    if (cudaStreamCreateWithFlags(&stage->stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&stage->done, cudaEventDisableTiming) != cudaSuccess)
      return fail(kCuda, "cannot create the context stream");
    std::size_t *arena = &stage->arena_bytes;
    EVOB_TRY(stage->allocate(&stage->hidden, T * D * 2, arena));
    EVOB_TRY(stage->allocate(&stage->residual, T * D * 2, arena));
    EVOB_TRY(stage->allocate(&stage->normalized, T * D * 2, arena));
    EVOB_TRY(stage->allocate(&stage->mixer_out, T * D * 2, arena));
    EVOB_TRY(stage->allocate(&stage->query, T * D * 2, arena));
    EVOB_TRY(stage->allocate(&stage->codes, T * D, arena));
    if (profile == ExecutionProfile::kTensorCoreFfn) {
      EVOB_TRY(stage_weights->ensure_fp8_ffn(c));
      EVOB_TRY(stage->allocate(&stage->codes_wide, T * I, arena));
      void *scales = nullptr;
      EVOB_TRY(stage->allocate(&scales, T * 4, arena));
      stage->row_scale = static_cast<float *>(scales);
    }
    EVOB_TRY(stage->allocate(&stage->projection, T * D * 6, arena));
    EVOB_TRY(stage->allocate(&stage->gated, T * I * 2, arena));
    if (!fused_gate) {
      EVOB_TRY(stage->allocate(&stage->mlp_first, T * I * 2, arena));
      EVOB_TRY(stage->allocate(&stage->mlp_second, T * I * 2, arena));
    }
    EVOB_TRY(stage->allocate(&stage->short_filtered, T * D * 6, arena));
    EVOB_TRY(stage->allocate(&stage->x2, T * D * 2, arena));
    EVOB_TRY(stage->allocate(&stage->x1, T * D * 2, arena));
    EVOB_TRY(stage->allocate(&stage->value, T * D * 2, arena));
    EVOB_TRY(stage->allocate(&stage->pregate, T * D * 2, arena));
    void *p = nullptr;
    EVOB_TRY(stage->allocate(&p, modal_scratch_floats(T, D, c.state_size) * 4 + 16, arena));
    stage->modal_scratch = static_cast<float *>(p);
    EVOB_TRY(stage->allocate(&p, T * 4, arena));
    stage->tokens = static_cast<std::uint32_t *>(p);
    EVOB_TRY(stage->allocate(&stage->logits, T * c.vocab * 2, arena));
    EVOB_TRY(stage->allocate(&stage->split_workspace, kSplitWorkspaceBytes, arena));
    stage->layers.resize(stage_weights->layers.size());
    std::size_t *cache = &stage->cache_bytes;
    for (std::size_t i = 0; i < stage->layers.size(); ++i) {
      LayerState &state = stage->layers[i];
      const MixerType type = stage_weights->layers[i].type;
      if (type == MixerType::kAttention && q8_kv) {
        state.q8_page_count = (context_size + kQ8PageTokens - 1) / kQ8PageTokens;
        EVOB_TRY(stage->allocate(&p, 4 * state.q8_page_count * sizeof(void *), cache));
        state.q8_tables = static_cast<void **>(p);
        if (cudaMemset(state.q8_tables, 0, 4 * state.q8_page_count * sizeof(void *)) != cudaSuccess)
          return fail(kCuda, "cannot clear the quantised KV page tables");
        if (stage->kv_image_key == nullptr) {
          EVOB_TRY(stage->allocate(&stage->kv_image_key, context_size * D * 2, cache));
          EVOB_TRY(stage->allocate(&stage->kv_image_value, context_size * D * 2, cache));
        }
        continue;
      }
      if (type == MixerType::kAttention) {
        EVOB_TRY(stage->allocate(&state.key_cache, context_size * D * 2, cache));
        EVOB_TRY(stage->allocate(&state.value_cache, context_size * D * 2, cache));
        continue;
      }
      EVOB_TRY(stage->allocate(&p, 3 * D * (c.short_taps - 1) * 4, cache));
      state.short_cache = static_cast<float *>(p);
      {
        const std::size_t taps = type == MixerType::kHcs ? c.hcs_taps
                                 : type == MixerType::kHcm ? c.hcm_taps : 1;
        // the fused kernels stage a 16-row-aligned halo plus the featurizer's two rows
        state.history_rows = std::min(kHistoryPad, (taps + 15) / 16 * 16 + (c.short_taps - 1));
        EVOB_TRY(stage->allocate(&state.history, state.history_rows * 3 * D * 2 + 16, cache));
        if (cudaMemset(state.history, 0, state.history_rows * 3 * D * 2) != cudaSuccess)
          return fail(kCuda, "cannot clear the projection history");
      }
      if (type == MixerType::kHcl) {
        EVOB_TRY(stage->allocate(&p, D * c.state_size * 4, cache));
        state.modal_state = static_cast<float *>(p);
      } else {
        const std::size_t taps = type == MixerType::kHcs ? c.hcs_taps : c.hcm_taps;
        EVOB_TRY(stage->allocate(&p, D * (taps - 1) * 4, cache));
        state.inner_cache = static_cast<float *>(p);
      }
    }
    context->stages_.push_back(std::move(stage));
  }
  {
    Stage &first = *context->stages_.front();
    DeviceGuard guard(first.device);
    void *p = nullptr;
    EVOB_TRY(first.allocate(&p, 16, &first.arena_bytes));
    context->device_position_ = static_cast<int *>(p);
    const char *const graphs = std::getenv("EVO_B200_DECODE_GRAPH");
    context->decode_graph_allowed_ = (graphs == nullptr || std::string(graphs) != "0") && !q8_kv;
    const char *const dependent = std::getenv("EVO_B200_DECODE_PDL");
    context->decode_dependent_launch_ = dependent == nullptr || std::string(dependent) != "0";
  }
  // Direct peer copies between neighbouring stages (and last -> first for the
  // head); without peer access the copies still work, staged by the driver.
  for (std::size_t i = 0; i < context->stages_.size() && context->stages_.size() > 1; ++i) {
    const int a = context->stages_[i]->device;
    const int b = context->stages_[(i + 1) % context->stages_.size()]->device;
    for (const auto &[from, to] : {std::pair<int, int>{a, b}, std::pair<int, int>{b, a}}) {
      int possible = 0;
      if (from == to || cudaDeviceCanAccessPeer(&possible, from, to) != cudaSuccess || !possible) continue;
      DeviceGuard guard(from);
      const cudaError_t error = cudaDeviceEnablePeerAccess(to, 0);
      if (error != cudaSuccess) cudaGetLastError();  // already enabled or refused: both fine
    }
  }
  *out = std::move(context);
  return kOk;
}

std::vector<StageAssignment> Context::stages() const {
  std::vector<StageAssignment> list;
  for (const auto &stage : stages_) {
    StageAssignment a;
    a.device = stage->device;
    a.layer_begin = stage->weights->layer_begin;
    a.layer_end = stage->weights->layer_end;
    a.weight_bytes = stage->weights->weight_bytes;
    a.cache_bytes = stage->cache_bytes;
    a.arena_bytes = stage->arena_bytes;
    list.push_back(a);
  }
  return list;
}

const void *Context::device_logits() const { return stages_.front()->logits; }
void *Context::first_stream() const { return stages_.front()->stream; }

int Context::synchronize() {
  int status = kOk;
  for (const auto &stage : stages_) {
    DeviceGuard guard(stage->device);
    if (cudaStreamSynchronize(stage->stream) != cudaSuccess) {
      status = fail(kCuda, std::string("stream synchronisation failed: ") +
                               cudaGetErrorString(cudaGetLastError()));
      break;
    }
    const int gemm = gemm_error_state(stage->stream);
    if (gemm != kOk) status = gemm;
    stage->collect_profile();
  }
  if (status != kOk) {
    healthy_ = false;
    state_valid_ = false;
  }
  return status;
}

const char *profile_category_name(const int category) {
  static const char *const names[kProfileCategories] = {
      "rms_norm", "gemm_bf16_tcgen05", "gemm_e4m3_tcgen05", "gemm_e4m3_emulated", "hcs_fused_fir",
      "hcm_fused_fir", "hcl_modal_scan", "attention", "state_step", "elementwise", "row_quantize",
      "gemm_e4m3_ffn_tcgen05"};
  return category >= 0 && category < kProfileCategories ? names[category] : "";
}

void Context::set_profiling(const bool enabled) {
  for (const auto &stage : stages_) {
    stage->profiling = enabled;
    if (enabled) {
      for (int i = 0; i < kProfileCategories; ++i) {
        stage->category_ms[i] = 0.0;
        stage->category_launches[i] = 0;
      }
    }
  }
}

void Context::read_profile(double (&milliseconds)[kProfileCategories],
                           std::uint64_t (&launches)[kProfileCategories]) const {
  for (int i = 0; i < kProfileCategories; ++i) {
    milliseconds[i] = 0.0;
    launches[i] = 0;
    for (const auto &stage : stages_) {
      milliseconds[i] += stage->category_ms[i];
      launches[i] += stage->category_launches[i];
    }
  }
}

// `window_begin` > 0 (Mode::kWindow) means: the stage's activation pointers have
// been advanced by window_begin rows by the caller and this call produces rows
// [window_begin, window_begin + rows) of a prefill whose earlier rows are still
// in the same arena buffers.  The fused Hyena kernels then read their history
// straight from those earlier rows.
int Context::run_stage(Stage &s, const std::size_t rows, const Mode mode,
                       const long capture_layer, std::vector<float> *captured,
                       const std::size_t window_begin, const std::size_t window_position,
                       const DumpPlan *const dumps) {
  const ModelConfig &c = weights_->config;
  const std::size_t D = c.width, I = c.inner_width;
  const bool window = mode == Mode::kWindow;
  const bool initial = mode == Mode::kPrefill || mode == Mode::kStateless ||
                       mode == Mode::kCachedPrefill || window;
  const bool stateless = mode == Mode::kStateless;
  const auto rewind = [&](void *advanced, const std::size_t row_bytes) -> void * {
    return static_cast<unsigned char *>(advanced) - window_begin * row_bytes;
  };
  cudaStream_t stream = s.stream;
  for (std::size_t i = 0; i < s.layers.size(); ++i) {
    const LayerWeights &w = s.weights->layers[i];
    LayerState &state = s.layers[i];
    const bool attention = w.type == MixerType::kAttention;
    const bool fp8 = !attention && c.fp8_projection;
    const std::size_t layer_index = s.weights->layer_begin + i;
    // taps of this block, if any were asked for (never in window mode)
    const DumpPlan *const tap = dumps != nullptr && dumps->wants_layer(layer_index) ? dumps : nullptr;
    const bool tap_pre_norm = tap != nullptr && tap->wants(layer_index, DumpPoint::kPreNorm);
    // pre-norm (+ E4M3 codes of the normalised activations for FP8 projections)
    EVOB_OP(kCatNorm, rms_norm(s.hidden, w.pre_norm, rows, D, c.epsilon,
                      fp8 && !tap_pre_norm ? nullptr : s.normalized, fp8 ? s.codes : nullptr,
                      w.projection_input_scale, stream));
    if (tap_pre_norm) EVOB_TRY(emit_bf16(stream, *tap, layer_index, DumpPoint::kPreNorm, s.normalized, rows, D));
    // input projection -> [rows, 3D]
    // prefill chunks of the FP8 FFN profile: output and MLP projections in E4M3 as well
    const bool ffn8 = profile_ == ExecutionProfile::kTensorCoreFfn && rows > 128 && w.out_codes != nullptr;
    if (fp8 && profile_ == ExecutionProfile::kExact) {
      EVOB_OP(kCatGemmEmulated, e4m3_emulated_gemm(s.codes, w.projection, rows, D, 3 * D,
                                  w.projection_output_scale, s.projection, stream));
    } else {
      LinearArgs a;
      a.split_workspace = s.split_workspace;
      a.split_workspace_bytes = kSplitWorkspaceBytes;
      a.dependent_launch = decode_dependent_launch_ && rows == 1;
      a.input = fp8 ? s.codes : s.normalized;
      a.weight = w.projection;
      a.output = s.projection;
      a.rows = rows;
      a.in_features = D;
      a.out_features = 3 * D;
      if (fp8) {
        a.operand_type = OperandType::kE4m3;
        a.alpha = w.projection_output_scale;
      }
      EVOB_OP(fp8 ? kCatGemmFp8 : kCatGemmBf16, linear(a, stream));
    }
    if (tap != nullptr)
      EVOB_TRY(emit_bf16(stream, *tap, layer_index, DumpPoint::kMixerInputProjection, s.projection, rows, 3 * D));
    if (attention) {
      const std::size_t prefix = window ? window_position : (initial ? 0 : position_);
      void *const keys = q8_kv_ ? s.kv_image_key : state.key_cache;
      void *const values = q8_kv_ ? s.kv_image_value : state.value_cache;
      if (q8_kv_) EVOB_TRY(s.ensure_q8_pages(state, prefix + rows, c.heads, c.head_dim()));
      EVOB_OP(kCatAttention, split_rope_append(s.projection, w.inverse_frequency, rows, c.heads, c.head_dim(),
                                 prefix, c.rope_scale, false, s.query, keys, values, context_size_, stream,
                                 mode == Mode::kDecode ? dynamic_position_ : nullptr));
      bool attended = false;
      if (q8_kv_) {
        // the new rows go into the pages as int8; what attention reads back is their quantised
        // value, for these rows as for every earlier one
        const Q8PageTable table = state.q8_table();
        EVOB_OP(kCatAttention, q8_kv_append(static_cast<unsigned char *>(keys) + prefix * D * 2,
                                            static_cast<unsigned char *>(values) + prefix * D * 2, table, prefix, rows,
                                            c.heads, c.head_dim(), stream));
        if (rows <= 8 && c.head_dim() == 128) {  // other head sizes attend to the BF16 image of the pages
          EVOB_OP(kCatAttention, q8_attention_decode(s.query, table, rows, prefix + rows, c.heads, c.head_dim(),
                                                     s.mixer_out, stream));
          attended = true;
        } else {
          EVOB_OP(kCatAttention, q8_kv_expand(table, prefix + rows, c.heads, c.head_dim(), keys, values, stream));
        }
      }
      if (tap != nullptr) {
        // rotated queries, and the rotated keys / values where the append left them in the cache
        EVOB_TRY(emit_bf16(stream, *tap, layer_index, DumpPoint::kMixerX2, s.query, rows, D));
        EVOB_TRY(emit_bf16(stream, *tap, layer_index, DumpPoint::kMixerX1,
                           static_cast<unsigned char *>(keys) + prefix * D * 2, rows, D));
        EVOB_TRY(emit_bf16(stream, *tap, layer_index, DumpPoint::kMixerValue,
                           static_cast<unsigned char *>(values) + prefix * D * 2, rows, D));
      }
      const bool cached = !q8_kv_ && (mode == Mode::kCachedPrefill ||
                                      ((mode == Mode::kDecode || mode == Mode::kContinue) && cached_attention_));
      if (attended) {
      } else if (cached)
        EVOB_OP(kCatAttention, cached_attention(s.query, keys, values, rows, prefix + rows,
                                  c.heads, c.head_dim(), s.mixer_out, stream));
      else
        EVOB_OP(kCatAttention, causal_attention(s.query, keys, values, rows, prefix + rows,
                                  c.heads, c.head_dim(), s.mixer_out, stream,
                                  mode == Mode::kDecode ? dynamic_position_ : nullptr));
    } else if (initial) {
      unsigned char *const projection_base =
          static_cast<unsigned char *>(rewind(s.projection, D * 6));
      if (window && window_position == 0 && window_begin > 0) {
        // first window of a sequence placed behind stale rows: its history is zeros
        const std::size_t have = std::min(state.history_rows, window_begin);
        if (cudaMemsetAsync(projection_base + (window_begin - have) * D * 6, 0, have * D * 6, stream) !=
            cudaSuccess)
          return fail(kCuda, "projection history clear failed");
      }
      if (window && state.history != nullptr && window_position > 0 && window_begin > 0) {
        // bring this block's own history back under the window
        const std::size_t have = std::min(state.history_rows, window_begin);
        if (cudaMemcpyAsync(projection_base + (window_begin - have) * D * 6,
                            static_cast<unsigned char *>(state.history) +
                                (state.history_rows - have) * D * 6,
                            have * D * 6, cudaMemcpyDeviceToDevice, stream) != cudaSuccess)
          return fail(kCuda, "projection history restore failed");
      }
      if (w.type == MixerType::kHcl) {
        ModalArgs a;
        a.projection = rewind(s.projection, D * 6);
        a.short_filter = w.short_filter;
        a.short_taps = c.short_taps;
        a.direct = w.direct;
        a.log_poles = w.log_poles;
        a.residues = w.residues;
        a.output = rewind(s.mixer_out, D * 2);
        a.state = stateless ? nullptr : state.modal_state;
        a.scratch = s.modal_scratch;
        a.short_cache = stateless ? nullptr : state.short_cache;
        a.length = window_begin + rows;
        a.row_begin = window_begin;
        a.continue_from_state = window && window_position > 0;
        a.width = D;
        a.modes = c.state_size;
        EVOB_OP(kCatModal, modal_prefill(a, stream));
      } else {
        const bool hcs = w.type == MixerType::kHcs;
        GatedFirArgs a;
        a.projection = rewind(s.projection, D * 6);
        a.short_filter = w.short_filter;
        a.short_taps = c.short_taps;
        a.filter = w.inner_filter;
        a.filter_is_f32 = !hcs && c.hcm_filter_f32;
        a.direct = hcs ? nullptr : w.direct;
        a.output = rewind(s.mixer_out, D * 2);
        a.length = window_begin + rows;
        a.row_begin = window_begin;
        a.width = D;
        a.groups = hcs ? c.hcs_groups : c.hcm_groups;
        a.taps = hcs ? c.hcs_taps : c.hcm_taps;
        a.cross_correlation = hcs;
        a.inner_cache = stateless ? nullptr : state.inner_cache;
        a.short_cache = stateless ? nullptr : state.short_cache;
        EVOB_OP(hcs ? kCatShortFir : kCatMediumFir, gated_fir_prefill(a, stream));
      }
      if (!window && !stateless && state.history != nullptr) {
        // leave the tail of this prompt as history for a later continuation chunk
        const std::size_t keep = std::min(state.history_rows, rows);
        if ((keep < state.history_rows &&
             cudaMemsetAsync(state.history, 0, (state.history_rows - keep) * D * 6, stream) != cudaSuccess) ||
            cudaMemcpyAsync(static_cast<unsigned char *>(state.history) + (state.history_rows - keep) * D * 6,
                            projection_base + (rows - keep) * D * 6, keep * D * 6, cudaMemcpyDeviceToDevice,
                            stream) != cudaSuccess)
          return fail(kCuda, "projection history save failed");
      }
      if (window && state.history != nullptr) {
        const std::size_t end = window_begin + rows;
        const std::size_t keep = std::min(state.history_rows, end);
        if (cudaMemcpyAsync(static_cast<unsigned char *>(state.history) +
                                (state.history_rows - keep) * D * 6,
                            projection_base + (end - keep) * D * 6, keep * D * 6,
                            cudaMemcpyDeviceToDevice, stream) != cudaSuccess)
          return fail(kCuda, "projection history save failed");
      }
    } else if (mode == Mode::kDecode && rows == 1 && c.short_taps == 3 && tap == nullptr &&
               position_ >= std::max({c.short_taps, c.hcs_taps, c.hcm_taps}) &&
               (w.type == MixerType::kHcl ? c.state_size <= 32 : (w.type == MixerType::kHcs ? c.hcs_taps : c.hcm_taps) <= 128)) {
      // one token against full histories: the whole mixer in one launch
      DecodeMixerArgs a;
      a.projection = s.projection;
      a.short_filter = w.short_filter;
      a.short_cache = state.short_cache;
      a.output = s.mixer_out;
      a.width = D;
      if (w.type == MixerType::kHcl) {
        a.direct = w.direct;
        a.log_poles = w.log_poles;
        a.residues = w.residues;
        a.modes = c.state_size;
        a.modal_state = state.modal_state;
      } else {
        const bool hcs = w.type == MixerType::kHcs;
        a.direct = hcs ? nullptr : w.direct;
        a.filter = w.inner_filter;
        a.filter_is_f32 = !hcs && c.hcm_filter_f32;
        a.groups = hcs ? c.hcs_groups : c.hcm_groups;
        a.taps = hcs ? c.hcs_taps : c.hcm_taps;
        a.cross_correlation = hcs;
        a.inner_cache = state.inner_cache;
      }
      EVOB_OP(kCatStateStep, hyena_decode_mixer(a, stream));
    } else {
      // continuation / decode against the causal state
      const std::size_t short_cached = std::min(position_, c.short_taps - 1);
      EVOB_OP(kCatStateStep, fir_step(s.projection, w.short_filter, false, nullptr, false, rows, 3 * D, 3 * D,
                        c.short_taps, true, state.short_cache, short_cached, s.short_filtered,
                        stream));
      EVOB_OP(kCatElementwise, split_triples(s.short_filtered, rows, D, s.x2, s.x1, s.value, stream));
      if (w.type == MixerType::kHcl) {
        if (mode == Mode::kDecode) {
          EVOB_OP(kCatStateStep, modal_decode(s.x2, s.x1, s.value, w.direct, w.log_poles, w.residues, D,
                                c.state_size, state.modal_state, s.pregate, s.mixer_out, stream));
        } else {
          ModalArgs a;
          a.x2 = s.x2;
          a.x1 = s.x1;
          a.value = s.value;
          a.direct = w.direct;
          a.log_poles = w.log_poles;
          a.residues = w.residues;
          a.output = s.mixer_out;
          a.pregate = tap != nullptr ? s.pregate : nullptr;
          a.state = state.modal_state;
          a.scratch = s.modal_scratch;
          a.length = rows;
          a.width = D;
          a.modes = c.state_size;
          a.continue_from_state = true;
          EVOB_OP(kCatModal, modal_prefill(a, stream));
        }
      } else {
        const bool hcs = w.type == MixerType::kHcs;
        const std::size_t taps = hcs ? c.hcs_taps : c.hcm_taps;
        EVOB_OP(kCatElementwise, gate(s.x1, s.value, s.pregate, rows * D, false, stream));
        EVOB_OP(kCatStateStep, fir_step(s.pregate, w.inner_filter, !hcs && c.hcm_filter_f32,
                          hcs ? nullptr : w.direct, !hcs, rows, D,
                          hcs ? c.hcs_groups : c.hcm_groups, taps, hcs, state.inner_cache,
                          std::min(position_, taps - 1), s.query, stream));
        EVOB_OP(kCatElementwise, gate(s.query, s.x2, s.mixer_out, rows * D, false, stream));
      }
    }
    if (tap != nullptr) {
      if (!attention) EVOB_TRY(dump_mixer_taps(s, i, rows, mode, *tap));
      EVOB_TRY(emit_bf16(stream, *tap, layer_index, DumpPoint::kMixerOutput, s.mixer_out, rows, D));
    }
    // output projection + bias + residual -> residual buffer
    {
      LinearArgs a;
      a.split_workspace = s.split_workspace;
      a.split_workspace_bytes = kSplitWorkspaceBytes;
      a.dependent_launch = decode_dependent_launch_ && rows == 1;
      a.input = s.mixer_out;
      a.weight = w.out_weight;
      a.bias = w.out_bias;
      a.residual = s.hidden;
      a.output = s.residual;
      a.rows = rows;
      a.in_features = D;
      a.out_features = D;
      // fused for attention and single-row Hyena, separately rounded otherwise
      // (upstream src/cuda/model.cu:1768-1799)
      a.bias_mode = (attention || rows == 1) ? 1 : 2;
      const bool out8 = ffn8 && (fp8_ffn_parts_ & 1U) != 0;
      if (out8) {
        EVOB_OP(kCatRowQuantize, quantize_rows(s.mixer_out, rows, D, s.codes, s.row_scale, stream));
        a.input = s.codes;
        a.weight = w.out_codes;
        a.operand_type = OperandType::kE4m3;
        a.alpha = w.out_dequant;
        a.row_scale = s.row_scale;
      }
      EVOB_OP(out8 ? kCatGemmFp8Ffn : kCatGemmBf16, linear(a, stream));
      if (tap != nullptr && tap->wants(layer_index, DumpPoint::kMixerProjection)) {
        // the projection before the residual joins it: the same product once more
        a.residual = nullptr;
        a.output = s.query;
        EVOB_TRY(linear(a, stream));
        EVOB_TRY(emit_bf16(stream, *tap, layer_index, DumpPoint::kMixerProjection, s.query, rows, D));
      }
    }
    if (tap != nullptr)
      EVOB_TRY(emit_bf16(stream, *tap, layer_index, DumpPoint::kMixerResidual, s.residual, rows, D));
    EVOB_OP(kCatNorm, rms_norm(s.residual, w.post_norm, rows, D, c.epsilon, s.normalized, nullptr, 1.0F,
                      stream));
    if (tap != nullptr)
      EVOB_TRY(emit_bf16(stream, *tap, layer_index, DumpPoint::kPostNorm, s.normalized, rows, D));
    const bool gelu_block = layer_index == 0;
    const bool up8 = ffn8 && (fp8_ffn_parts_ & 2U) != 0, down8 = ffn8 && (fp8_ffn_parts_ & 4U) != 0;
    if (w.l12 != nullptr) {
      LinearArgs a;
      a.split_workspace = s.split_workspace;
      a.split_workspace_bytes = kSplitWorkspaceBytes;
      a.dependent_launch = decode_dependent_launch_ && rows == 1;
      a.input = s.normalized;
      a.weight = w.l12;
      a.output = s.gated;
      a.rows = rows;
      a.in_features = D;
      a.out_features = 2 * I;
      a.gate_mode = gelu_block ? 2 : 1;
      if (up8) {
        EVOB_OP(kCatRowQuantize, quantize_rows(s.normalized, rows, D, s.codes, s.row_scale, stream));
        a.input = s.codes;
        a.weight = w.l12_codes;
        a.operand_type = OperandType::kE4m3;
        a.alpha = w.l12_dequant;
        a.row_scale = s.row_scale;
      }
      EVOB_OP(up8 ? kCatGemmFp8Ffn : kCatGemmBf16, linear(a, stream));
    } else {
      LinearArgs a;
      a.split_workspace = s.split_workspace;
      a.split_workspace_bytes = kSplitWorkspaceBytes;
      a.input = s.normalized;
      a.rows = rows;
      a.in_features = D;
      a.out_features = I;
      a.weight = w.l1;
      a.output = s.mlp_first;
      EVOB_OP(kCatGemmBf16, linear(a, stream));
      a.weight = w.l2;
      a.output = s.mlp_second;
      EVOB_OP(kCatGemmBf16, linear(a, stream));
      EVOB_OP(kCatElementwise, gate(s.mlp_first, s.mlp_second, s.gated, rows * I, gelu_block, stream));
    }
    if (tap != nullptr) {
      EVOB_TRY(dump_mlp_taps(s, i, rows, up8, *tap));
      EVOB_TRY(emit_bf16(stream, *tap, layer_index, DumpPoint::kMlpGated, s.gated, rows, I));
    }
    {
      LinearArgs a;
      a.split_workspace = s.split_workspace;
      a.split_workspace_bytes = kSplitWorkspaceBytes;
      a.dependent_launch = decode_dependent_launch_ && rows == 1;
      a.input = s.gated;
      a.weight = w.l3;
      a.residual = s.residual;
      a.output = s.hidden;
      a.rows = rows;
      a.in_features = I;
      a.out_features = D;
      if (down8) {
        EVOB_OP(kCatRowQuantize, quantize_rows(s.gated, rows, I, s.codes_wide, s.row_scale, stream));
        a.input = s.codes_wide;
        a.weight = w.l3_codes;
        a.operand_type = OperandType::kE4m3;
        a.alpha = w.l3_dequant;
        a.row_scale = s.row_scale;
      }
      EVOB_OP(down8 ? kCatGemmFp8Ffn : kCatGemmBf16, linear(a, stream));
      if (tap != nullptr && tap->wants(layer_index, DumpPoint::kMlpOutput)) {
        a.residual = nullptr;
        a.output = s.query;
        EVOB_TRY(linear(a, stream));
        EVOB_TRY(emit_bf16(stream, *tap, layer_index, DumpPoint::kMlpOutput, s.query, rows, D));
      }
    }
    if (tap != nullptr)
      EVOB_TRY(emit_bf16(stream, *tap, layer_index, DumpPoint::kBlockOutput, s.hidden, rows, D));
    if (capture_layer >= 0 && static_cast<std::size_t>(capture_layer) == layer_index &&
        captured != nullptr) {
      std::vector<std::uint16_t> raw(rows * D);
      if (cudaMemcpyAsync(raw.data(), s.hidden, raw.size() * 2, cudaMemcpyDeviceToHost, stream) !=
              cudaSuccess ||
          cudaStreamSynchronize(stream) != cudaSuccess)
        return fail(kCuda, "layer capture failed");
      captured->resize(raw.size());
      for (std::size_t j = 0; j < raw.size(); ++j) {
        const std::uint32_t bits = static_cast<std::uint32_t>(raw[j]) << 16U;
        std::memcpy(&(*captured)[j], &bits, 4);
      }
    }
  }
  return kOk;
}

int Context::run_wavefront(const std::size_t rows, const Mode /*mode*/, const long /*capture_layer*/,
                           std::vector<float> * /*captured*/) {
  const ModelConfig &c = weights_->config;
  const std::size_t D = c.width, I = c.inner_width;
  std::size_t chunk = wavefront_chunk_;
  if (chunk == 0) {
    // enough chunks to fill the pipeline (about two per stage up to four stages, one per
    // stage beyond), none so small that the tensor-core tiles run half empty
    const std::size_t per_stage = stages_.size() <= 4 ? 2 : 1;
    chunk = (rows / (per_stage * stages_.size()) + 255) / 256 * 256;
    chunk = std::max<std::size_t>(512, std::min<std::size_t>(chunk, 2048));
  }
  for (std::size_t begin = 0; begin < rows; begin += chunk) {
    const std::size_t count = std::min(chunk, rows - begin);
    for (std::size_t index = 0; index < stages_.size(); ++index) {
      Stage &stage = *stages_[index];
      DeviceGuard guard(stage.device);
      if (index > 0) {
        Stage &previous = *stages_[index - 1];
        // the wait binds to the record of this chunk on the previous stage,
        // issued just before; later records of the same event do not affect it
        if (cudaStreamWaitEvent(stage.stream, previous.done, 0) != cudaSuccess ||
            cudaMemcpyPeerAsync(static_cast<unsigned char *>(stage.hidden) + begin * D * 2, stage.device,
                                static_cast<unsigned char *>(previous.hidden) + begin * D * 2,
                                previous.device, count * D * 2, stage.stream) != cudaSuccess)
          return fail(kCuda, "stage hand-off failed");
      }
      stage.shift_rows(static_cast<long>(begin), D, I);
      const int status = run_stage(stage, count, Mode::kWindow, -1, nullptr, begin, begin);
      stage.shift_rows(-static_cast<long>(begin), D, I);
      if (status != kOk) return status;
      if (cudaEventRecord(stage.done, stage.stream) != cudaSuccess)
        return fail(kCuda, "stage hand-off failed");
    }
  }
  return kOk;
}

int Context::forward(const std::uint32_t *host_tokens, const std::uint32_t *device_tokens,
                     const std::size_t rows, const Mode mode, std::vector<float> *logits,
                     const long capture_layer, std::vector<float> *captured, const DumpPlan *const dumps) {
  const ModelConfig &c = weights_->config;
  if (!healthy_) return fail(kInvalidArgument, "context was invalidated by an earlier failure");
  if (weights_->slice_count > 1)
    return fail(kInvalidArgument, "this model holds one pipeline slice: drive it with the slice calls");
  if (rows == 0 || rows > arena_rows_)
    return fail(kInvalidArgument, "model forward arguments are invalid");
  const bool initial = mode == Mode::kPrefill || mode == Mode::kStateless || mode == Mode::kCachedPrefill;
  if (initial) {
    if (rows > context_size_) return fail(kInvalidArgument, "prompt exceeds the context capacity");
  } else if (!state_valid_ || position_ > context_size_ || rows > context_size_ - position_ ||
             (mode == Mode::kDecode && rows != 1)) {
    return fail(kInvalidArgument,
                "continuation requires a valid prefill and free context capacity");
  }
  if (host_tokens != nullptr)
    for (std::size_t i = 0; i < rows; ++i)
      if (host_tokens[i] >= c.vocab)
        return fail(kInvalidArgument, "token ID exceeds model vocabulary");
  int status = kOk;
  Stage &first = *stages_.front();
  // A continuation chunk of more than a few rows runs through the fused
  // prefill kernels as a row window: its rows sit kHistoryPad rows into the
  // activation buffers and every Hyena block puts its own last projection rows
  // in front of them.  (Short chunks and the exact cached-attention profile
  // keep the step kernels.)
  const bool continuation_window = mode == Mode::kContinue && rows >= 16 && !cached_attention_ &&
                                   capture_layer < 0 && history_current_ && dumps == nullptr;
  struct ShiftBack {
    Context *context;
    bool active;
    ~ShiftBack() {
      if (!active) return;
      const ModelConfig &config = context->weights_->config;
      for (auto &stage : context->stages_)
        stage->shift_rows(-static_cast<long>(kHistoryPad), config.width, config.inner_width);
    }
  } shift_back{this, continuation_window};
  if (continuation_window)
    for (auto &stage : stages_) stage->shift_rows(static_cast<long>(kHistoryPad), c.width, c.inner_width);
  bool graph_step = false;
  if (decode_graph_allowed_ && mode == Mode::kDecode && stages_.size() == 1 && host_tokens != nullptr &&
      !first.profiling && !cached_attention_ && c.head_dim() == 128 && capture_layer < 0 &&
      dumps == nullptr && position_ >= std::max({c.short_taps, c.hcs_taps, c.hcm_taps}))
    status = decode_step_graph(host_tokens, &graph_step);
  if (!graph_step && status == kOk) {
    DeviceGuard guard(first.device);
    if (host_tokens != nullptr) {
      if (cudaMemcpyAsync(first.tokens, host_tokens, rows * 4, cudaMemcpyHostToDevice,
                          first.stream) != cudaSuccess)
        status = fail(kCuda, "token upload failed");
      device_tokens = first.tokens;
    }
    if (status == kOk)
      status = embedding(device_tokens, first.weights->embedding, rows, c.width, c.vocab, first.hidden,
                         first.stream);
  }
  const bool wavefront = stages_.size() > 1 && (mode == Mode::kPrefill || mode == Mode::kStateless) &&
                         rows >= 512 && capture_layer < 0 && dumps == nullptr;
  if (wavefront && status == kOk) status = run_wavefront(rows, mode, capture_layer, captured);
  for (std::size_t index = 0; index < stages_.size() && status == kOk && !wavefront && !graph_step; ++index) {
    Stage &stage = *stages_[index];
    DeviceGuard guard(stage.device);
    if (index > 0) {
      Stage &previous = *stages_[index - 1];
      if (cudaStreamWaitEvent(stage.stream, previous.done, 0) != cudaSuccess ||
          cudaMemcpyPeerAsync(stage.hidden, stage.device, previous.hidden, previous.device,
                              rows * c.width * 2, stage.stream) != cudaSuccess)
        status = fail(kCuda, "stage hand-off failed");
    }
    if (status == kOk)
      status = continuation_window
                   ? run_stage(stage, rows, Mode::kWindow, -1, nullptr, kHistoryPad, position_)
                   : run_stage(stage, rows, mode, capture_layer, captured, 0, 0, dumps);
    if (status == kOk && cudaEventRecord(stage.done, stage.stream) != cudaSuccess)
      status = fail(kCuda, "stage hand-off failed");
  }
  if (status == kOk) {
    DeviceGuard guard(first.device);
    if (stages_.size() > 1) {
      Stage &last = *stages_.back();
      if (cudaStreamWaitEvent(first.stream, last.done, 0) != cudaSuccess ||
          cudaMemcpyPeerAsync(first.hidden, first.device, last.hidden, last.device,
                              rows * c.width * 2, first.stream) != cudaSuccess)
        status = fail(kCuda, "stage hand-off failed");
    }
    if (status == kOk && !graph_step)
      status = rms_norm(first.hidden, first.weights->final_norm, rows, c.width, c.epsilon,
                        first.normalized, nullptr, 1.0F, first.stream);
    if (status == kOk && !graph_step) {
      LinearArgs a;
      a.split_workspace = first.split_workspace;
      a.split_workspace_bytes = kSplitWorkspaceBytes;
      a.dependent_launch = decode_dependent_launch_ && rows == 1;
      a.input = first.normalized;
      a.weight = first.weights->embedding;  // tied head
      a.output = first.logits;
      a.rows = rows;
      a.in_features = c.width;
      a.out_features = c.vocab;
      status = linear(a, first.stream);
    }
    if (status == kOk && logits != nullptr) {
      std::vector<std::uint16_t> raw(rows * c.vocab);
      if (cudaMemcpyAsync(raw.data(), first.logits, raw.size() * 2, cudaMemcpyDeviceToHost,
                          first.stream) != cudaSuccess ||
          cudaStreamSynchronize(first.stream) != cudaSuccess) {
        status = fail(kCuda, std::string("logits read-back failed: ") +
                                 cudaGetErrorString(cudaGetLastError()));
      } else {
        logits->resize(raw.size());
        for (std::size_t j = 0; j < raw.size(); ++j) {
          const std::uint32_t bits = static_cast<std::uint32_t>(raw[j]) << 16U;
          std::memcpy(&(*logits)[j], &bits, 4);
        }
        for (const auto &stage : stages_) {
          DeviceGuard stage_guard(stage->device);
          if (status == kOk) status = gemm_error_state(stage->stream);
          stage->collect_profile();
        }
      }
    }
  }
  if (status != kOk) {
    state_valid_ = false;
    healthy_ = false;
    return status;
  }
  const bool stateless = mode == Mode::kStateless;
  // the per-block projection history is written by the fused prefill kernels only: steps taken
  // with the step kernels (decode, short continuations) leave it behind the sequence
  history_current_ = (initial && !stateless) || continuation_window;
  position_ = stateless ? 0 : (initial ? rows : position_ + rows);
  state_valid_ = !stateless;
  if (initial) cached_attention_ = mode == Mode::kCachedPrefill;
  return kOk;
}

// Sequence position p of a sliced context lives at row kHistoryPad +
// p % activation_capacity of the activation buffers: windows of a prompt that
// fits the arena keep distinct rows (sends of earlier windows may still be in
// flight), longer prompts wrap around, and every Hyena block finds room for its
// carried history in front of the window.  slice_hidden() points at the row of
// position 0.
void *Context::slice_hidden() const {
  return static_cast<unsigned char *>(stages_.front()->hidden) + kHistoryPad * weights_->config.width * 2;
}

int Context::slice_embed(const std::uint32_t *device_tokens, const std::size_t position,
                         const std::size_t rows) {
  Stage &stage = *stages_.front();
  if (!healthy_) return fail(kInvalidArgument, "context was invalidated by an earlier failure");
  const std::size_t offset = position % arena_rows_;
  if (device_tokens == nullptr || rows == 0 || offset + rows > arena_rows_ ||
      stage.weights->embedding == nullptr || stage.weights->layer_begin != 0)
    return fail(kInvalidArgument, "slice_embed needs the first slice, a token buffer and a window inside the arena");
  DeviceGuard guard(stage.device);
  return embedding(device_tokens, stage.weights->embedding, rows, weights_->config.width,
                   weights_->config.vocab,
                   static_cast<unsigned char *>(stage.hidden) + (kHistoryPad + offset) * weights_->config.width * 2,
                   stage.stream);
}

int Context::slice_run(const std::size_t position, const std::size_t rows) {
  const ModelConfig &c = weights_->config;
  Stage &stage = *stages_.front();
  if (!healthy_) return fail(kInvalidArgument, "context was invalidated by an earlier failure");
  if (stages_.size() != 1 || weights_->slice_count < 2)
    return fail(kInvalidArgument, "slice_run needs a model loaded as one slice of a pipeline");
  const std::size_t offset = position % arena_rows_;
  if (rows == 0 || offset + rows > arena_rows_ || position + rows > context_size_ ||
      (position != 0 && position != position_))
    return fail(kInvalidArgument,
                "slice windows must be contiguous, ascending, inside the context and not straddle the arena");
  DeviceGuard guard(stage.device);
  state_valid_ = false;  // decode across processes is not provided
  const std::size_t first_row = kHistoryPad + offset;
  stage.shift_rows(static_cast<long>(first_row), c.width, c.inner_width);
  const int status = run_stage(stage, rows, Mode::kWindow, -1, nullptr, first_row, position);
  stage.shift_rows(-static_cast<long>(first_row), c.width, c.inner_width);
  if (status != kOk) {
    healthy_ = false;
    return status;
  }
  position_ = position + rows;
  return kOk;
}

int Context::slice_head(const std::size_t position, const std::size_t rows) {
  const ModelConfig &c = weights_->config;
  Stage &stage = *stages_.front();
  if (!healthy_) return fail(kInvalidArgument, "context was invalidated by an earlier failure");
  const std::size_t offset = position % arena_rows_;
  if (rows == 0 || offset + rows > arena_rows_ || stage.weights->embedding == nullptr ||
      stage.weights->layer_end != c.layers)
    return fail(kInvalidArgument, "slice_head needs the last slice and a window inside the arena");
  DeviceGuard guard(stage.device);
  unsigned char *const hidden = static_cast<unsigned char *>(stage.hidden) + (kHistoryPad + offset) * c.width * 2;
  unsigned char *const normalized =
      static_cast<unsigned char *>(stage.normalized) + (kHistoryPad + offset) * c.width * 2;
  int status = rms_norm(hidden, stage.weights->final_norm, rows, c.width, c.epsilon, normalized, nullptr,
                        1.0F, stage.stream);
  if (status != kOk) return status;
  LinearArgs a;
  a.split_workspace = stage.split_workspace;
  a.split_workspace_bytes = kSplitWorkspaceBytes;
  a.input = normalized;
  a.weight = stage.weights->embedding;  // tied head
  a.output = static_cast<unsigned char *>(stage.logits) + offset * c.vocab * 2;
  a.rows = rows;
  a.in_features = c.width;
  a.out_features = c.vocab;
  return linear(a, stage.stream);
}

int Context::prefill(const std::vector<std::uint32_t> &tokens, std::vector<float> *logits) {
  if (logits == nullptr) return fail(kInvalidArgument, "logits output is null");
  return forward(tokens.data(), nullptr, tokens.size(), Mode::kPrefill, logits, -1, nullptr);
}
int Context::prefill_stateless(const std::vector<std::uint32_t> &tokens, std::vector<float> *logits) {
  if (logits == nullptr) return fail(kInvalidArgument, "logits output is null");
  return forward(tokens.data(), nullptr, tokens.size(), Mode::kStateless, logits, -1, nullptr);
}
int Context::prefill_cached(const std::vector<std::uint32_t> &tokens, std::vector<float> *logits) {
  if (logits == nullptr) return fail(kInvalidArgument, "logits output is null");
  return forward(tokens.data(), nullptr, tokens.size(), Mode::kCachedPrefill, logits, -1, nullptr);
}
int Context::prefill_chunk(const std::vector<std::uint32_t> &tokens, std::vector<float> *logits) {
  if (logits == nullptr) return fail(kInvalidArgument, "logits output is null");
  if (state_valid_ && cached_attention_)
    return fail(kInvalidArgument, "a cached prefill continues through exact token decode only, not through another chunk");
  return forward(tokens.data(), nullptr, tokens.size(), Mode::kContinue, logits, -1, nullptr);
}
int Context::decode(const std::uint32_t token, std::vector<float> *logits) {
  if (logits == nullptr) return fail(kInvalidArgument, "logits output is null");
  return forward(&token, nullptr, 1, Mode::kDecode, logits, -1, nullptr);
}
int Context::prefill_embedding(const std::vector<std::uint32_t> &tokens, const std::size_t layer,
                               std::vector<float> *hidden) {
  if (hidden == nullptr || layer >= weights_->config.layers)
    return fail(kInvalidArgument, "layer capture index or output is invalid");
  std::vector<float> logits;
  return forward(tokens.data(), nullptr, tokens.size(), Mode::kStateless, &logits,
                 static_cast<long>(layer), hidden);
}
int Context::prefill_chunk_embedding(const std::vector<std::uint32_t> &tokens, const std::size_t layer,
                                     const bool first, std::vector<float> *hidden) {
  if (hidden == nullptr || layer >= weights_->config.layers)
    return fail(kInvalidArgument, "layer capture index or output is invalid");
  if (!first && state_valid_ && cached_attention_)
    return fail(kInvalidArgument, "a cached prefill continues through exact token decode only, not through another chunk");
  std::vector<float> logits;
  return forward(tokens.data(), nullptr, tokens.size(), first ? Mode::kPrefill : Mode::kContinue, &logits,
                 static_cast<long>(layer), hidden);
}
int Context::prefill_with_dumps(const std::vector<std::uint32_t> &tokens, const DumpPlan &plan,
                                const bool cached, std::vector<float> *logits) {
  if (logits == nullptr) return fail(kInvalidArgument, "logits output is null");
  for (const DumpPlan::Request &request : plan.requests)
    if (request.layer >= weights_->config.layers || static_cast<int>(request.point) < 0 ||
        request.point >= DumpPoint::kDumpPoints)
      return fail(kInvalidArgument, "CUDA dump layer is out of range");
  return forward(tokens.data(), nullptr, tokens.size(), cached ? Mode::kCachedPrefill : Mode::kPrefill, logits, -1,
                 nullptr, &plan);
}
int Context::decode_with_dumps(const std::uint32_t token, const DumpPlan &plan, std::vector<float> *logits) {
  if (logits == nullptr) return fail(kInvalidArgument, "logits output is null");
  for (const DumpPlan::Request &request : plan.requests)
    if (request.layer >= weights_->config.layers || static_cast<int>(request.point) < 0 ||
        request.point >= DumpPoint::kDumpPoints)
      return fail(kInvalidArgument, "CUDA dump layer is out of range");
  return forward(&token, nullptr, 1, Mode::kDecode, logits, -1, nullptr, &plan);
}
int Context::continue_device(const std::uint32_t *device_tokens, const std::size_t rows) {
  if (device_tokens == nullptr) return fail(kInvalidArgument, "token buffer is null");
  if (state_valid_ && cached_attention_)
    return fail(kInvalidArgument, "a cached prefill continues through exact token decode only, not through another chunk");
  return forward(nullptr, device_tokens, rows, Mode::kContinue, nullptr, -1, nullptr);
}
int Context::prefill_device(const std::uint32_t *device_tokens, const std::size_t rows,
                            const bool stateless) {
  if (device_tokens == nullptr) return fail(kInvalidArgument, "token buffer is null");
  return forward(nullptr, device_tokens, rows, stateless ? Mode::kStateless : Mode::kPrefill,
                 nullptr, -1, nullptr);
}

}  // namespace evob
