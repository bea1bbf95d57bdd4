// StripedHyena2 runtime: configuration, device-resident weights, per-context
// state and the layer pipeline.  Mirrors the public surface of upstream's
// evo::cuda::PipelineModel (include/evo/cuda/model.hpp:107-229): load,
// shared-weight contexts, prefill / stateless / cached prefill, chunk
// continuation, decode, layer capture, stage reporting.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "safetensors.hpp"

namespace evob {

enum class MixerType { kHcs, kHcm, kHcl, kAttention };

// Operator classes reported by the optional per-operator timing.
enum ProfileCategory : int {
  kCatNorm = 0,        // RMSNorm (+ fused E4M3 quantisation)
  kCatGemmBf16,        // tcgen05 BF16 projections (Wqkv, out, MLP, head)
  kCatGemmFp8,         // tcgen05 E4M3 Hyena projections
  kCatGemmEmulated,    // bit-exact software-QGMMA Hyena projections
  kCatShortFir,        // HCS (k=7) fused featurizer + FIR + gates
  kCatMediumFir,       // HCM (k=128) fused featurizer + FIR + gates
  kCatModal,           // HCL modal scan
  kCatAttention,       // QKV split/RoPE/append + attention
  kCatStateStep,       // continuation / decode FIR and state updates
  kCatElementwise,     // embedding, gates, splits
  kCatRowQuantize,     // per-row E4M3 quantisation in front of the FP8 FFN / output projections
  kCatGemmFp8Ffn,      // tcgen05 E4M3 output and MLP projections (profile b200-fp8)
  kProfileCategories
};
const char *profile_category_name(int category);

// Named activation taps inside a block, in upstream's order and with
// upstream's names (LayerDumpPoint, include/evo/cuda/model.hpp:22-45).
enum class DumpPoint : int {
  kBlockOutput = 0, kPreNorm, kMixerInputProjection, kMixerShortFilter, kMixerShortState,
  kMixerInnerState, kMixerX2, kMixerX1, kMixerValue, kMixerPregate, kMixerState, kMixerFilter,
  kMixerConvolution, kMixerOutput, kMixerProjection, kMixerResidual, kPostNorm, kMlpL1, kMlpL2,
  kMlpActivation, kMlpGated, kMlpOutput, kDumpPoints
};
const char *dump_point_name(int point);  // "block_output", "pre_norm", ... ; "" when out of range

// A set of (layer, point) taps and the consumer of their values.  The sink
// gets F32 values [rows, columns] (BF16 buffers widened) that are valid during
// the call; a non-zero return aborts the forward pass with that status.
struct DumpPlan {
  struct Request {
    std::size_t layer = 0;
    DumpPoint point = DumpPoint::kBlockOutput;
  };
  std::vector<Request> requests;
  std::function<int(const Request &request, const float *values, std::size_t rows, std::size_t columns)> sink;
  bool wants(std::size_t layer, DumpPoint point) const {
    for (const Request &r : requests)
      if (r.layer == layer && r.point == point) return true;
    return false;
  }
  bool wants_layer(std::size_t layer) const {
    for (const Request &r : requests)
      if (r.layer == layer) return true;
    return false;
  }
};

// How E4M3 Hyena projections are evaluated.  kExact reproduces upstream's
// software-QGMMA rounding bit for bit; kTensorCore uses tcgen05 FP8 MMAs with
// F32 accumulation (its own execution profile, tolerance parity).
// kTensorCoreFfn additionally runs the output and MLP projections of prefill
// chunks in E4M3 with dynamic per-row activation scales (profile "b200-fp8").
enum class ExecutionProfile { kExact, kTensorCore, kTensorCoreFfn };

struct ModelConfig {
  std::string architecture, model_id, model_name, artifact_profile;
  bool test_fixture = false;
  std::size_t vocab = 0, width = 0, layers = 0, heads = 0, state_size = 0, inner_width = 0;
  std::size_t short_taps = 0, hcs_taps = 0, hcm_taps = 0, hcs_groups = 0, hcm_groups = 0;
  std::size_t max_seqlen = 0;
  float epsilon = 1e-6F, rope_scale = 1.0F, rope_base = 10000.0F;
  bool fp8_projection = false, hcm_filter_f32 = false, qkv_source_head_major = false;
  std::vector<MixerType> mixers;  // one per block
  std::size_t head_dim() const { return width / heads; }
};

int read_model_config(const ModelFile &file, bool allow_test_fixture, ModelConfig *config);
// Every tensor the configuration calls for is there with its type and shape, and nothing else is
// (host only; load_weights makes the same checks while it gathers the views).
int check_tensor_set(const ModelFile &file, const ModelConfig &config);

struct LayerWeights {
  MixerType type = MixerType::kHcs;
  const float *pre_norm = nullptr, *post_norm = nullptr;
  const void *projection = nullptr;  // [3D, D] BF16 or E4M3 codes (Wqkv for attention)
  float projection_input_scale = 1.0F, projection_output_scale = 1.0F;
  const void *short_filter = nullptr;   // [3D, short_taps] BF16
  const void *inner_filter = nullptr;   // [groups, taps] BF16 or F32
  const void *direct = nullptr;         // [D] BF16 (HCM, HCL)
  const float *log_poles = nullptr, *residues = nullptr;  // [D, S]
  const float *inverse_frequency = nullptr;               // [head_dim/2]
  const void *out_weight = nullptr, *out_bias = nullptr;  // [D, D], [D]
  const void *l1 = nullptr, *l2 = nullptr, *l3 = nullptr;
  const void *l12 = nullptr;  // row-interleaved [2I, D] for the fused gate GEMM
  std::size_t payload_bytes = 0;
  // E4M3 copies for the FP8 FFN profile (StageWeights::ensure_fp8_ffn): codes in the
  // layout of the BF16 tensor, and 1 / (448 / max|w|) for the epilogue.
  const void *out_codes = nullptr, *l12_codes = nullptr, *l3_codes = nullptr;
  float out_dequant = 1.0F, l12_dequant = 1.0F, l3_dequant = 1.0F;
};

// Immutable device weights of one pipeline stage (one GPU).
struct StageWeights {
  int device = 0;
  std::size_t layer_begin = 0, layer_end = 0;
  std::vector<LayerWeights> layers;
  const void *embedding = nullptr;    // stage 0 (and the last slice of a per-process pipeline)
  const float *final_norm = nullptr;  // same
  void *slab = nullptr;
  std::size_t slab_bytes = 0, weight_bytes = 0;
  // Quantises the output / MLP projection weights of every block once (first
  // context of the FP8 FFN profile); later calls return at once.  Thread-safe.
  int ensure_fp8_ffn(const ModelConfig &config);
  void *ffn_slab = nullptr;
  std::size_t ffn_slab_bytes = 0;
  ~StageWeights();
};

struct ModelWeights {
  ModelConfig config;
  std::vector<std::shared_ptr<StageWeights>> stages;
  // Per-process pipelines: this process holds stage `slice_index` of
  // `slice_count` (one StageWeights); 0 / 1 for a model held by one process.
  std::size_t slice_index = 0, slice_count = 1;
};

struct StageAssignment {
  int device = 0;
  std::size_t layer_begin = 0, layer_end = 0;
  std::size_t weight_bytes = 0, cache_bytes = 0, arena_bytes = 0;
};

// Contiguous byte-balanced split of `layers` blocks over `stage_count` stages
// (upstream src/cuda/model.cu:2419-2469); host-only, unit-testable.
std::vector<std::pair<std::size_t, std::size_t>> plan_stages(
    const std::vector<std::size_t> &layer_bytes, std::size_t stage_count, bool even_split);

int load_weights(const ModelFile &file, const std::vector<int> &devices,
                 bool allow_test_fixture, std::size_t layer_limit,
                 std::shared_ptr<ModelWeights> *out, std::size_t slice_index = 0,
                 std::size_t slice_count = 1);

class Context {
 public:
  ~Context();
  // q8_kv: keys and values are kept as per-vector int8 in lazily allocated pages of 16,384
  // tokens (upstream's fast-q8-kv profile, docs/execution-profiles.md:96-127).  Any head size: steps of
  // 1..8 rows read the pages directly at head size 128, everything else attends to their BF16 image.
  static int create(std::shared_ptr<ModelWeights> weights, std::size_t context_size,
                    ExecutionProfile profile, bool full_arena_for_fixtures,
                    std::unique_ptr<Context> *out, bool q8_kv = false);

  // logits: rows * vocab floats (converted from BF16).
  int prefill(const std::vector<std::uint32_t> &tokens, std::vector<float> *logits);
  int prefill_stateless(const std::vector<std::uint32_t> &tokens, std::vector<float> *logits);
  int prefill_cached(const std::vector<std::uint32_t> &tokens, std::vector<float> *logits);
  int prefill_chunk(const std::vector<std::uint32_t> &tokens, std::vector<float> *logits);
  int decode(std::uint32_t token, std::vector<float> *logits);
  // Block output of `layer` ([rows, width] floats) for a fresh stateless prefill.
  int prefill_embedding(const std::vector<std::uint32_t> &tokens, std::size_t layer,
                        std::vector<float> *hidden);
  // Chunked form (upstream prefill_embedding / prefill_chunk_embedding,
  // include/evo/cuda/model.hpp:150-170): the first chunk starts the sequence, later ones continue it;
  // the context advances like a prefill.
  int prefill_chunk_embedding(const std::vector<std::uint32_t> &tokens, std::size_t layer, bool first,
                              std::vector<float> *hidden);
  // Upstream's prefill_with_dumps / prefill_cached_with_dumps / decode_with_dumps
  // (include/evo/cuda/model.hpp:121-134, 184-190): the same passes with the
  // requested taps handed to plan.sink as they are produced.  A layer with taps
  // inside its mixer or MLP runs the unfused operator sequence for those taps
  // next to the fused kernels, so that every intermediate exists as a buffer;
  // the block's own results still come from the ordinary path.
  int prefill_with_dumps(const std::vector<std::uint32_t> &tokens, const DumpPlan &plan, bool cached,
                         std::vector<float> *logits);
  int decode_with_dumps(std::uint32_t token, const DumpPlan &plan, std::vector<float> *logits);

  // Device-resident variant used by the benchmark: tokens already on the
  // device of stage 0, logits left on the device (BF16 [rows, vocab]).
  int prefill_device(const std::uint32_t *device_tokens, std::size_t rows, bool stateless);
  // Next chunk of the same sequence, same conventions (needs a non-stateless prefill before).
  int continue_device(const std::uint32_t *device_tokens, std::size_t rows);
  const void *device_logits() const;
  void *first_stream() const;

  // ---- one stage of a pipeline spread over processes (slice_count > 1).
  // The launcher moves hidden rows between processes (NCCL send/recv straight
  // from / into slice_hidden()); each call below enqueues on the stage stream
  // and returns.  Rows are produced window by window in ascending order:
  //   slice 0:      slice_embed(tokens, b, n); slice_run(b, n); send rows
  //   slice i:      receive rows; slice_run(b, n); send rows
  //   last slice:   receive rows; slice_run(b, n); ... slice_head(0, total)
  int slice_embed(const std::uint32_t *device_tokens, std::size_t row_begin, std::size_t rows);
  int slice_run(std::size_t row_begin, std::size_t rows);
  int slice_head(std::size_t row_begin, std::size_t rows);
  void *slice_hidden() const;  // [activation_capacity, width] BF16
  std::size_t slice_index() const { return weights_->slice_index; }
  std::size_t slice_count() const { return weights_->slice_count; }
  // Waits for every stage stream and surfaces asynchronous kernel errors.
  int synchronize();
  // Per-operator timing (CUDA events around every launch; adds a few
  // microseconds per operator, so keep it off for throughput measurements).
  void set_profiling(bool enabled);
  // Totals accumulated since profiling was enabled, summed over stages.
  void read_profile(double (&milliseconds)[kProfileCategories],
                    std::uint64_t (&launches)[kProfileCategories]) const;

  std::size_t position() const { return position_; }
  std::size_t activation_capacity() const { return arena_rows_; }
  std::size_t context_capacity() const { return context_size_; }
  const ModelConfig &config() const { return weights_->config; }
  ExecutionProfile profile() const { return profile_; }
  std::vector<StageAssignment> stages() const;
  bool shares_weights_with(const Context &other) const { return weights_ == other.weights_; }
  bool poisoned() const { return !healthy_; }
  bool uses_q8_kv_cache() const { return q8_kv_; }

 private:
  struct Stage;
  enum class Mode { kPrefill, kStateless, kCachedPrefill, kContinue, kDecode, kWindow };
  Context() = default;
  int forward(const std::uint32_t *host_tokens, const std::uint32_t *device_tokens,
              std::size_t rows, Mode mode, std::vector<float> *logits, long capture_layer,
              std::vector<float> *captured, const DumpPlan *dumps = nullptr);
  int run_stage(Stage &stage, std::size_t rows, Mode mode, long capture_layer,
                std::vector<float> *captured, std::size_t window_begin = 0,
                std::size_t window_position = 0, const DumpPlan *dumps = nullptr);
  // Taps of block `layer` of `stage` (dumps.cu-style helpers in model.cu).
  int dump_mixer_taps(Stage &stage, std::size_t local_layer, std::size_t rows, Mode mode,
                      const DumpPlan &dumps);
  int dump_mlp_taps(Stage &stage, std::size_t local_layer, std::size_t rows, bool fp8_ffn,
                    const DumpPlan &dumps);
  // Chunk wavefront over the pipeline stages: chunk j runs on stage s while
  // chunk j+1 runs on stage s-1 (legal because every mixer carries causal
  // state).  Used for initial prefills on more than one stage.
  int run_wavefront(std::size_t rows, Mode mode, long capture_layer, std::vector<float> *captured);
  std::size_t wavefront_chunk_ = 0;  // 0 = choose from rows and stage count
  // Cached decode as a replayed CUDA graph (single-stage contexts, head size
  // 128, history full; EVO_B200_DECODE_GRAPH=0 turns it off).
  int decode_step_graph(const std::uint32_t *host_token, bool *launched);
  void *decode_graph_ = nullptr;          // cudaGraphExec_t
  int *device_position_ = nullptr;        // position of the decoded token, read by replayed kernels
  const int *dynamic_position_ = nullptr; // == device_position_ while the graph is being recorded
  int decode_position_host_ = 0;
  bool decode_graph_allowed_ = true;
  // one-row projections are launched with programmatic stream serialisation (EVO_B200_DECODE_PDL=0: plain launches)
  bool decode_dependent_launch_ = true;

  std::shared_ptr<ModelWeights> weights_;
  std::vector<std::unique_ptr<Stage>> stages_;
  ExecutionProfile profile_ = ExecutionProfile::kExact;
  // Which projections the FP8 FFN profile quantises: bit 0 output projection, bit 1 MLP
  // up-projections, bit 2 MLP down-projection (EVO_B200_FP8_FFN_PARTS, default all).
  unsigned fp8_ffn_parts_ = 7U;
  bool q8_kv_ = false;
  std::size_t context_size_ = 0, arena_rows_ = 0, position_ = 0;
  bool state_valid_ = false, cached_attention_ = false, healthy_ = true;
  bool history_current_ = false;  // per-block projection history covers the rows up to position_
};

}  // namespace evob
