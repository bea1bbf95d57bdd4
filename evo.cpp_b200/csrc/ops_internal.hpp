// Host-side launchers of the sm_100a kernels.  All pointers are device
// pointers on the current device; every function returns an evo_status value
// and records a message retrievable through evob::last_error().
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace evob {

// ---- fp8_codec.cpp: host E4M3FN codec (upstream include/evo/fp8.hpp)
namespace fp8 {
std::uint8_t encode_e4m3fn(float value) noexcept;
float decode_e4m3fn(std::uint8_t code) noexcept;
bool valid_scale(float scale) noexcept;
float scaled_e4m3fn_roundtrip(float value, float scale) noexcept;
}  // namespace fp8

// ---- elementwise.cu
int quantize_bf16(const void *input, std::size_t elements, float scale,
                  void *codes, float *dequantized, cudaStream_t stream);
int quantize_f32(const float *input, std::size_t elements, float scale,
                 void *codes, cudaStream_t stream);
// Per-row dynamic quantisation of a BF16 matrix: codes[r, :] = E4M3(x[r, :] * q_r)
// with q_r = 448 / max|x[r, :]| (1 for an all-zero row) and row_scale[r] = 1 / q_r.
int quantize_rows(const void *input, std::size_t rows, std::size_t width, void *codes,
                  float *row_scale, cudaStream_t stream);
// Largest magnitude of a BF16 tensor, left on the device as a BF16 bit pattern.
int amax_bf16(const void *input, std::size_t elements, unsigned int *result_bits, cudaStream_t stream);
int rms_norm(const void *input, const float *scale, std::size_t rows,
             std::size_t width, float epsilon, void *output, void *codes,
             float quant_scale, cudaStream_t stream,
             // few rows only: launch with programmatic stream serialisation (the gains are fetched under the
             // kernel in front, the row after it has finished).  The decode step does not ask for it: with the
             // norm released early the projection behind it starts two kernels ahead and its waiting CTAs take
             // SM slots from the projection still running (2.63 against 2.59 ms per token).
             bool dependent_launch = false);
int gelu(const void *input, void *output, std::size_t elements,
         cudaStream_t stream);
int gate(const void *first, const void *second, void *output,
         std::size_t elements, bool apply_gelu, cudaStream_t stream);
int add(const void *first, const void *second, void *output,
        std::size_t elements, cudaStream_t stream);
int add_bias(void *output, const void *bias, std::size_t rows,
             std::size_t width, cudaStream_t stream);
// Ids >= vocabulary are not looked up: the row becomes zeros and the per-device
// error word is raised (reported by gemm_error_state as an invalid argument).
int embedding(const std::uint32_t *tokens, const void *table, std::size_t rows,
              std::size_t width, std::size_t vocabulary, void *output,
              cudaStream_t stream);
int split_triples(const void *projection, std::size_t rows, std::size_t width,
                  void *x2, void *x1, void *value, cudaStream_t stream);
int transpose(const void *input, std::size_t rows, std::size_t columns,
              void *output, cudaStream_t stream);

// ---- qgmma_emulation.cu
int e4m3_emulated_gemm(const void *input_codes, const void *weight_codes,
                       std::size_t rows, std::size_t in_features,
                       std::size_t out_features, float output_scale,
                       void *output, cudaStream_t stream);

// ---- gemm_tcgen05.cu
enum class OperandType { kBf16, kE4m3 };
struct LinearArgs {
  const void *input = nullptr;   // [rows, in_features] BF16 or E4M3 codes
  const void *weight = nullptr;  // [out_features, in_features], same type
  const void *bias = nullptr;    // [out_features] BF16
  const void *residual = nullptr;  // [rows, out_features] BF16
  void *output = nullptr;        // [rows, out_features (/2 when gated)] BF16
  std::size_t rows = 0;
  std::size_t in_features = 0;
  std::size_t out_features = 0;
  OperandType operand_type = OperandType::kBf16;
  float alpha = 1.0F;  // applied to the F32 accumulator before rounding
  // Optional per-row factor [rows] F32 (tile kernel only): the accumulator of row r
  // is multiplied by alpha * row_scale[r] (dynamic per-row activation quantisation).
  const float *row_scale = nullptr;
  // One-row weight streams only: launch with programmatic stream serialisation, so that the kernel may
  // start (and pull its weights into L2) while the kernel in front of it in the stream is still running;
  // it waits for that kernel before it reads the input.  The caller promises that nothing this launch
  // reads besides `weight` is still being written by work further back than the previous kernel.
  bool dependent_launch = false;
  int bias_mode = 0;   // 0 none, 1 fused F32 add, 2 separate BF16-rounded add
  int gate_mode = 0;   // 0 none, 1 a*b, 2 gelu(a)*b over 128-column halves
  bool force_simt = false;
  // F32-result mode (BF16 operands, tensor-core path only): the F32 accumulator
  // times alpha, plus bias_f32, is stored (or added) to output_f32 [rows,
  // out_features] without any BF16 rounding.  weight_wrap_features = W makes the
  // weight's K coordinate wrap every W input features, so an input that is
  // several planes side by side, [x0 | x1 | ...] with in_features = planes * W,
  // is multiplied against the same [out_features, W] weight: the sum of the
  // planes' products in one accumulator.
  // Optional scratch for split-K at <= 32 rows (the projection is then a weight
  // stream and needs more CTAs than it has output tiles): F32 partial sums,
  // up to 8 * rows * out_features floats are used when they fit.  Owned by the
  // caller, one per stream.
  void *split_workspace = nullptr;
  std::size_t split_workspace_bytes = 0;
  float *output_f32 = nullptr;
  const float *bias_f32 = nullptr;
  bool accumulate_f32 = false;
  std::size_t weight_wrap_features = 0;
};
int linear(const LinearArgs &args, cudaStream_t stream);
// gemv.cu: weight-streaming kernel that linear() uses for 1..8 rows.
bool small_batch_linear_applicable(const LinearArgs &args);
int small_batch_linear(const LinearArgs &args, cudaStream_t stream);
// Synchronises the stream and reports (then clears) the per-device sticky error
// word: bit 0 = a pipeline wait of a tcgen05 kernel timed out (cuda), bit 1 = a
// device-resident token id was outside the vocabulary (invalid_argument).
int gemm_error_state(cudaStream_t stream);
// The word itself, for kernels that raise it.
int *device_error_word(int *status);

// ---- hyena_fir.cu
struct GatedFirArgs {
  // Either three separate [length, width] tensors ...
  const void *x2 = nullptr;
  const void *x1 = nullptr;
  const void *value = nullptr;
  // ... or the raw projection [length, 3*width] (interleaved x2,x1,v triples)
  // plus the per-stream 3-tap featurizer filter [3*width, short_taps].
  const void *projection = nullptr;
  const void *short_filter = nullptr;
  std::size_t short_taps = 0;
  const void *filter = nullptr;   // [groups, taps] BF16 or F32
  bool filter_is_f32 = false;
  const void *direct = nullptr;   // [width] BF16, adds direct*u (HCM) or null
  void *output = nullptr;         // [length, width] BF16
  void *pregate = nullptr;        // optional [length, width] BF16 (u = x1*v)
  std::size_t length = 0;
  // Rows [row_begin, length) are produced; rows before row_begin are history
  // that is still present in the same input buffers (chunked prefill inside
  // one activation arena).
  std::size_t row_begin = 0;
  std::size_t width = 0;
  std::size_t groups = 0;
  std::size_t taps = 0;
  bool cross_correlation = true;  // HCS: true, HCM: false
  // Optional F32 caches written for later decode steps.
  float *inner_cache = nullptr;   // [width, taps-1]
  float *short_cache = nullptr;   // [3*width, short_taps-1]
};
// Dispatches to the vectorised / tensor-core kernels of hyena_fir_fused.cu
// when the layout allows and to the generic kernel of hyena_fir.cu otherwise.
int gated_fir_prefill(const GatedFirArgs &args, cudaStream_t stream);
int gated_fir_prefill_generic(const GatedFirArgs &args, cudaStream_t stream);
// hyena_fir_tcgen05.cu: the k <= 128 causal-convolution form on tcgen05 tensor cores (projection-fed,
// BF16 filters shared by groups of exactly 16 channels); gated_fir_prefill uses it when applicable.
bool gated_fir_tcgen05_applicable(const GatedFirArgs &args);
int gated_fir_tcgen05(const GatedFirArgs &args, cudaStream_t stream);

int fir_prefill(const void *input, const void *filter, bool filter_is_f32,
                const void *bias, bool multiply_bias, std::size_t length,
                std::size_t channels, std::size_t groups, std::size_t taps,
                bool cross_correlation, void *output, float *cache,
                cudaStream_t stream);
int fill_fir_cache(const void *input, float *cache, std::size_t length,
                   std::size_t channels, std::size_t cache_size,
                   cudaStream_t stream);
int fir_step(const void *input, const void *filter, bool filter_is_f32,
             const void *bias, bool multiply_bias, std::size_t length,
             std::size_t channels, std::size_t groups, std::size_t taps,
             bool cross_correlation, float *cache, std::size_t cache_length,
             void *output, cudaStream_t stream);

// ---- hyena_modal.cu
struct ModalArgs {
  const void *x2 = nullptr;
  const void *x1 = nullptr;
  const void *value = nullptr;
  const void *projection = nullptr;
  const void *short_filter = nullptr;
  std::size_t short_taps = 0;
  const void *direct = nullptr;      // [width] BF16
  const float *log_poles = nullptr;  // [width, modes]
  const float *residues = nullptr;   // [width, modes]
  void *output = nullptr;            // [length, width] BF16
  void *pregate = nullptr;           // optional u
  float *state = nullptr;            // [width, modes] F32 in/out (may be null)
  float *scratch = nullptr;          // segment states, see modal_scratch_floats
  float *short_cache = nullptr;
  std::size_t length = 0;
  std::size_t row_begin = 0;  // rows [row_begin, length) are produced (see GatedFirArgs)
  std::size_t width = 0;
  std::size_t modes = 0;
  bool continue_from_state = false;  // recurrence-continue numerics
};
std::size_t modal_scratch_floats(std::size_t length, std::size_t width,
                                 std::size_t modes);
int modal_prefill(const ModalArgs &args, cudaStream_t stream);
// Same operator with its segment-state scratch in a fixed array inside the
// library image instead of args.scratch (which is ignored); separate x2/x1/v
// inputs only.  Makes no device allocation.
int modal_prefill_static_scratch(const ModalArgs &args, cudaStream_t stream);
// Diagnostic taps: the time-domain modal filter [length, width] F32 and / or
// the unrounded convolution of `gated` ([length, width] BF16, u = x1 * v) with it
// from a zero state; either output may be null.
int modal_taps(const void *gated, const float *log_poles, const float *residues, std::size_t length,
               std::size_t width, std::size_t modes, float *filter, float *convolution,
               cudaStream_t stream);
// One cached-decode step of a whole Hyena mixer (featurizer step, split, gate,
// inner FIR or modal step with their cache updates, post-gate) in one launch;
// bit-identical to the unfused sequence.  All histories must be full.  Set
// log_poles for the modal (HCL) form, filter for the FIR (HCS / HCM) forms.
struct DecodeMixerArgs {
  const void *projection = nullptr;    // [3 width] BF16, (x2, x1, v) per channel
  const void *short_filter = nullptr;  // [3 width, 3] BF16
  float *short_cache = nullptr;        // [3 width, 2] F32, advanced
  const void *direct = nullptr;        // [width] BF16 (HCM, HCL)
  const void *filter = nullptr;        // [groups, taps]
  bool filter_is_f32 = false;
  std::size_t groups = 0, taps = 0;
  bool cross_correlation = false;
  float *inner_cache = nullptr;        // [width, taps-1] F32, advanced
  const float *log_poles = nullptr, *residues = nullptr;  // [width, modes]
  std::size_t modes = 0;
  float *modal_state = nullptr;        // [width, modes] F32, advanced
  void *output = nullptr;              // [width] BF16
  std::size_t width = 0;
};
int hyena_decode_mixer(const DecodeMixerArgs &args, cudaStream_t stream);
int modal_decode(const void *x2, const void *x1, const void *value,
                 const void *direct, const float *log_poles,
                 const float *residues, std::size_t width, std::size_t modes,
                 float *state, void *pregate, void *output,
                 cudaStream_t stream);

// ---- kv_q8.cu: quantised KV cache (profile fast-q8-kv)
// Device arrays of page pointers; page p holds positions [p * page_tokens, (p + 1) * page_tokens):
// codes [page_tokens, heads, 128] int8 and scales [page_tokens, heads] F32.
struct Q8PageTable {
  std::int8_t *const *key = nullptr;
  std::int8_t *const *value = nullptr;
  float *const *key_scale = nullptr;
  float *const *value_scale = nullptr;
  std::size_t page_tokens = 0;
};
// K, V: BF16 [rows, heads, head_dim] of positions first_position ..; the pages must exist.
int q8_kv_append(const void *key, const void *value, const Q8PageTable &pages, std::size_t first_position,
                 std::size_t rows, std::size_t heads, std::size_t head_dim, cudaStream_t stream);
// BF16 images [count, heads, head_dim] of positions [0, count).
int q8_kv_expand(const Q8PageTable &pages, std::size_t count, std::size_t heads, std::size_t head_dim, void *key,
                 void *value, cudaStream_t stream);
// Decode attention (1..8 query rows, head size 128) straight from the pages; same contract as
// causal_attention.
int q8_attention_decode(const void *query, const Q8PageTable &pages, std::size_t rows, std::size_t total_keys,
                        std::size_t heads, std::size_t head_dim, void *output, cudaStream_t stream);

// ---- attention.cu
int split_rope_append(const void *qkv, const float *inverse_frequency,
                      std::size_t rows, std::size_t heads,
                      std::size_t head_dim, std::size_t position_offset,
                      float position_scale, bool head_major, void *query,
                      void *key_cache, void *value_cache,
                      std::size_t cache_capacity, cudaStream_t stream,
                      const int *dynamic_position = nullptr);
// dynamic_position / dynamic_prefix (optional, device int): the position of the
// first row, read by the kernel at run time instead of the host value - for
// launches recorded once and replayed (CUDA graphs).  Only the small-row kernels
// take it.
int causal_attention(const void *query, const void *key_cache,
                     const void *value_cache, std::size_t rows,
                     std::size_t total_keys, std::size_t heads,
                     std::size_t head_dim, void *output, cudaStream_t stream,
                     const int *dynamic_prefix = nullptr);
// Warp-level MMA / row-wise implementation of the same contract (what
// causal_attention falls back to below 128 rows or for other head sizes).
int causal_attention_mma_sync(const void *query, const void *key_cache,
                              const void *value_cache, std::size_t rows,
                              std::size_t total_keys, std::size_t heads,
                              std::size_t head_dim, void *output, cudaStream_t stream);
int cached_attention(const void *query, const void *key_cache,
                     const void *value_cache, std::size_t rows,
                     std::size_t total_keys, std::size_t heads,
                     std::size_t head_dim, void *output, cudaStream_t stream,
                     void *probabilities = nullptr);  // optional BF16 [heads, rows, total_keys]

// ---- linear_executor.cu: dense-linear offload with upstream's LinearExecutor contract
struct LinearExecutorState;
int linear_executor_create(int device, LinearExecutorState **out);
void linear_executor_free(LinearExecutorState *state);
std::size_t linear_executor_cached_bytes(LinearExecutorState *state);
int linear_executor_linear(LinearExecutorState *state, const float *input, std::size_t rows,
                           std::size_t input_width, const void *weight, int weight_dtype,
                           std::size_t weight_elements, std::size_t output_width, const void *bias,
                           int bias_dtype, std::size_t bias_elements, float *output);

}  // namespace evob
