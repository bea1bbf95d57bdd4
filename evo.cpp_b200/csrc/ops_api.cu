// extern "C" operator entry points declared in include/evo_b200_ops.h.
#include "../../include/evo_b200_ops.h"

#include "common.cuh"
#include "ops_internal.hpp"

namespace {

using namespace evob;

cudaStream_t as_stream(void *stream) { return static_cast<cudaStream_t>(stream); }

// Row-interleave W1/W2 in blocks of 128 rows so that every 256-column GEMM
// tile holds matching halves of both up-projections.
__global__ void interleave_gate_kernel(const uint4 *__restrict__ w1,
                                       const uint4 *__restrict__ w2,
                                       uint4 *__restrict__ out,
                                       const std::size_t inner,
                                       const std::size_t vectors_per_row) {
  const std::size_t total = inner * 2 * vectors_per_row;
  const std::size_t stride = static_cast<std::size_t>(blockDim.x) * gridDim.x;
  for (std::size_t i = static_cast<std::size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
       i < total; i += stride) {
    const std::size_t row = i / vectors_per_row, v = i % vectors_per_row;
    const std::size_t tile = row / 256, within = row % 256;
    const std::size_t source = tile * 128 + within % 128;
    out[i] = (within < 128 ? w1 : w2)[source * vectors_per_row + v];
  }
}

int fp8_linear(const bool tensor_core, const void *input, const void *weight,
               const std::size_t rows, const std::size_t in_features,
               const std::size_t out_features, const float input_scale,
               const float output_scale, void *scratch, void *output,
               cudaStream_t stream) {
  if (scratch == nullptr)
    return fail(kInvalidArgument, "software E4M3 linear needs a code workspace");
  if (in_features % 32 != 0)
    return fail(kInvalidArgument,
                "software E4M3 linear needs K to be a multiple of 32");
  int status = quantize_bf16(input, rows * in_features, input_scale, scratch,
                             nullptr, stream);
  if (status != kOk) return status;
  if (!tensor_core)
    return e4m3_emulated_gemm(scratch, weight, rows, in_features, out_features,
                              output_scale, output, stream);
  LinearArgs args;
  args.input = scratch;
  args.weight = weight;
  args.output = output;
  args.rows = rows;
  args.in_features = in_features;
  args.out_features = out_features;
  args.operand_type = OperandType::kE4m3;
  args.alpha = output_scale;
  return linear(args, stream);
}

}  // namespace

extern "C" {

const char *evo_b200_last_error(void) { return evob::last_error(); }

int evo_b200_check_async_errors(void *stream) {
  return gemm_error_state(as_stream(stream));
}

int evo_b200_software_e4m3_quantize_bf16(const void *input, size_t elements,
                                         float scale, void *codes,
                                         float *dequantized, void *stream) {
  return quantize_bf16(input, elements, scale, codes, dequantized, as_stream(stream));
}

int evo_b200_software_e4m3_quantize_f32_codes(const float *input,
                                              size_t elements, float scale,
                                              void *codes, void *stream) {
  return quantize_f32(input, elements, scale, codes, as_stream(stream));
}

int evo_b200_software_e4m3_h100_linear(const void *input, const void *weight,
                                       size_t rows, size_t in_features,
                                       size_t out_features, float input_scale,
                                       float output_scale, void *scratch,
                                       void *output, void *stream) {
  return fp8_linear(false, input, weight, rows, in_features, out_features,
                    input_scale, output_scale, scratch, output, as_stream(stream));
}

int evo_b200_e4m3_tensorcore_linear(const void *input, const void *weight,
                                    size_t rows, size_t in_features,
                                    size_t out_features, float input_scale,
                                    float output_scale, void *scratch,
                                    void *output, void *stream) {
  return fp8_linear(true, input, weight, rows, in_features, out_features,
                    input_scale, output_scale, scratch, output, as_stream(stream));
}

int evo_b200_e4m3_quantize_rows(const void *input, size_t rows, size_t width, void *codes_u8, float *row_scale,
                                void *stream) {
  return quantize_rows(input, rows, width, codes_u8, row_scale, as_stream(stream));
}

int evo_b200_e4m3_codes_linear(const void *input_codes, const float *row_scale, const void *weight_codes,
                               const void *bias, const void *residual, size_t rows, size_t in_features,
                               size_t out_features, float alpha, int bias_mode, int gate_mode, void *output,
                               void *stream) {
  LinearArgs args;
  args.input = input_codes;
  args.weight = weight_codes;
  args.operand_type = OperandType::kE4m3;
  args.row_scale = row_scale;
  args.alpha = alpha;
  args.bias = bias;
  args.residual = residual;
  args.output = output;
  args.rows = rows;
  args.in_features = in_features;
  args.out_features = out_features;
  args.bias_mode = bias == nullptr ? 0 : bias_mode;
  args.gate_mode = gate_mode;
  if (bias != nullptr && bias_mode != 1 && bias_mode != 2)
    return fail(kInvalidArgument, "linear bias mode must be 1 or 2");
  if (gate_mode < 0 || gate_mode > 2) return fail(kInvalidArgument, "gate mode must be 0, 1 or 2");
  return linear(args, as_stream(stream));
}

int evo_b200_bf16_linear(const void *input, const void *weight,
                         const void *bias, const void *residual, size_t rows,
                         size_t in_features, size_t out_features,
                         int bias_mode, int path, void *output, void *stream) {
  LinearArgs args;
  args.input = input;
  args.weight = weight;
  args.bias = bias;
  args.residual = residual;
  args.output = output;
  args.rows = rows;
  args.in_features = in_features;
  args.out_features = out_features;
  args.bias_mode = bias == nullptr ? 0 : bias_mode;
  args.force_simt = path == 1;
  if (bias != nullptr && bias_mode != 1 && bias_mode != 2)
    return fail(kInvalidArgument, "linear bias mode must be 1 or 2");
  return linear(args, as_stream(stream));
}

int evo_b200_bf16_linear_split_k(const void *input, const void *weight, const void *bias,
                                 const void *residual, size_t rows, size_t in_features,
                                 size_t out_features, int bias_mode, int gate_mode,
                                 void *workspace, size_t workspace_bytes, void *output,
                                 void *stream) {
  if (gate_mode < 0 || gate_mode > 2) return fail(kInvalidArgument, "gate mode must be 0, 1 or 2");
  if (bias != nullptr && bias_mode != 1 && bias_mode != 2)
    return fail(kInvalidArgument, "linear bias mode must be 1 or 2");
  LinearArgs args;
  args.input = input;
  args.weight = weight;
  args.bias = bias;
  args.residual = residual;
  args.output = output;
  args.rows = rows;
  args.in_features = in_features;
  args.out_features = out_features;
  args.bias_mode = bias == nullptr ? 0 : bias_mode;
  args.gate_mode = gate_mode;
  args.split_workspace = workspace;
  args.split_workspace_bytes = workspace_bytes;
  return linear(args, as_stream(stream));
}

int evo_b200_bf16_gated_up_projection(const void *input, const void *weight,
                                      size_t rows, size_t in_features,
                                      size_t inner_width, int activation,
                                      void *output, void *stream) {
  if (inner_width % 128 != 0)
    return fail(kInvalidArgument,
                "fused gated projection needs an inner width that is a "
                "multiple of 128");
  LinearArgs args;
  args.input = input;
  args.weight = weight;
  args.output = output;
  args.rows = rows;
  args.in_features = in_features;
  args.out_features = inner_width * 2;
  args.gate_mode = activation == 1 ? 2 : 1;
  return linear(args, as_stream(stream));
}

int evo_b200_interleave_gate_weights(const void *w1, const void *w2,
                                     size_t inner_width, size_t in_features,
                                     void *interleaved, void *stream) {
  if (w1 == nullptr || w2 == nullptr || interleaved == nullptr ||
      inner_width % 128 != 0 || in_features % 8 != 0 || in_features == 0)
    return fail(kInvalidArgument, "gate weight interleave arguments are invalid");
  if (inner_width == 0) return kOk;
  interleave_gate_kernel<<<kSmCount * 8, 256, 0, as_stream(stream)>>>(
      static_cast<const uint4 *>(w1), static_cast<const uint4 *>(w2),
      static_cast<uint4 *>(interleaved), inner_width, in_features / 8);
  return check_launch("gate weight interleave kernel");
}

int evo_b200_bf16_rms_norm(const void *input, const float *scale, size_t rows,
                           size_t width, float epsilon, void *output,
                           void *codes, float quant_scale, void *stream) {
  return rms_norm(input, scale, rows, width, epsilon, output, codes,
                  quant_scale, as_stream(stream));
}

int evo_b200_bf16_gelu(const void *input, size_t elements, void *output,
                       void *stream) {
  return gelu(input, output, elements, as_stream(stream));
}

int evo_b200_bf16_gated_elementwise(const void *first, const void *second,
                                    size_t elements, int apply_gelu,
                                    void *output, void *stream) {
  return gate(first, second, output, elements, apply_gelu != 0, as_stream(stream));
}

int evo_b200_bf16_add(const void *first, const void *second, size_t elements,
                      void *output, void *stream) {
  return add(first, second, output, elements, as_stream(stream));
}

int evo_b200_bf16_add_bias_inplace(void *output, const void *bias, size_t rows,
                                   size_t width, void *stream) {
  return add_bias(output, bias, rows, width, as_stream(stream));
}

int evo_b200_bf16_row_to_column_major(const void *input, size_t rows,
                                      size_t columns, void *output,
                                      void *stream) {
  return transpose(input, rows, columns, output, as_stream(stream));
}

int evo_b200_embedding(const uint32_t *tokens, const void *table, size_t rows,
                       size_t width, size_t vocabulary, void *output, void *stream) {
  return embedding(tokens, table, rows, width, vocabulary, output, as_stream(stream));
}

int evo_b200_bf16_split_hyena_projection(const void *projection, size_t rows,
                                         size_t width, void *x2, void *x1,
                                         void *value, void *stream) {
  return split_triples(projection, rows, width, x2, x1, value, as_stream(stream));
}

int evo_b200_bf16_fir_prefill_direct(const void *input, const void *filter,
                                     int filter_is_f32, const void *bias,
                                     size_t length, size_t channels,
                                     size_t groups, size_t taps,
                                     int orientation, int bias_mode,
                                     void *output, float *cache, void *stream) {
  return fir_prefill(input, filter, filter_is_f32 != 0, bias, bias_mode == 1,
                     length, channels, groups, taps, orientation == 0, output,
                     cache, as_stream(stream));
}

int evo_b200_bf16_fir_continue_direct(const void *input, const void *filter,
                                      int filter_is_f32, const void *bias,
                                      size_t length, size_t channels,
                                      size_t groups, size_t taps,
                                      int orientation, int bias_mode,
                                      float *cache, size_t cache_length,
                                      void *output, void *stream) {
  return fir_step(input, filter, filter_is_f32 != 0, bias, bias_mode == 1,
                  length, channels, groups, taps, orientation == 0, cache,
                  cache_length, output, as_stream(stream));
}

int evo_b200_bf16_hyena_decode_mixer(const void *projection, const void *short_filter, float *short_cache,
                                     const void *direct, const void *filter, int filter_is_f32,
                                     size_t groups, size_t taps, int orientation, float *inner_cache,
                                     const float *log_poles, const float *residues, size_t modes,
                                     float *modal_state, size_t width, void *output, void *stream) {
  DecodeMixerArgs a;
  a.projection = projection;
  a.short_filter = short_filter;
  a.short_cache = short_cache;
  a.direct = direct;
  a.filter = filter;
  a.filter_is_f32 = filter_is_f32 != 0;
  a.groups = groups;
  a.taps = taps;
  a.cross_correlation = orientation == 0;
  a.inner_cache = inner_cache;
  a.log_poles = log_poles;
  a.residues = residues;
  a.modes = modes;
  a.modal_state = modal_state;
  a.width = width;
  a.output = output;
  return hyena_decode_mixer(a, as_stream(stream));
}

int evo_b200_bf16_gated_fir_prefill(const void *x2, const void *x1,
                                    const void *value, const void *filter,
                                    int filter_is_f32, const void *direct,
                                    size_t length, size_t width, size_t groups,
                                    size_t taps, int orientation, void *pregate,
                                    float *inner_cache, void *output,
                                    void *stream) {
  GatedFirArgs a;
  a.x2 = x2;
  a.x1 = x1;
  a.value = value;
  a.filter = filter;
  a.filter_is_f32 = filter_is_f32 != 0;
  a.direct = direct;
  a.length = length;
  a.width = width;
  a.groups = groups;
  a.taps = taps;
  a.cross_correlation = orientation == 0;
  a.pregate = pregate;
  a.inner_cache = inner_cache;
  a.output = output;
  return gated_fir_prefill(a, as_stream(stream));
}

int evo_b200_bf16_gated_fir_prefill_window(const void *x2, const void *x1, const void *value,
                                           const void *filter, int filter_is_f32,
                                           const void *direct, size_t row_begin, size_t length,
                                           size_t width, size_t groups, size_t taps,
                                           int orientation, float *inner_cache, void *output,
                                           void *stream) {
  GatedFirArgs a;
  a.x2 = x2;
  a.x1 = x1;
  a.value = value;
  a.filter = filter;
  a.filter_is_f32 = filter_is_f32 != 0;
  a.direct = direct;
  a.row_begin = row_begin;
  a.length = length;
  a.width = width;
  a.groups = groups;
  a.taps = taps;
  a.cross_correlation = orientation == 0;
  a.inner_cache = inner_cache;
  a.output = output;
  return gated_fir_prefill(a, as_stream(stream));
}

int evo_b200_bf16_hcl_prefill_window(const void *x2, const void *x1, const void *value,
                                     const void *direct, const float *log_poles,
                                     const float *residues, size_t row_begin, size_t length,
                                     size_t width, size_t modes, float *state, float *scratch,
                                     void *output, void *stream) {
  ModalArgs a;
  a.x2 = x2;
  a.x1 = x1;
  a.value = value;
  a.direct = direct;
  a.log_poles = log_poles;
  a.residues = residues;
  a.row_begin = row_begin;
  a.length = length;
  a.width = width;
  a.modes = modes;
  a.continue_from_state = true;
  a.state = state;
  a.scratch = scratch;
  a.output = output;
  return modal_prefill(a, as_stream(stream));
}

int evo_b200_bf16_projection_gated_fir_prefill(
    const void *projection, const void *short_filter, const void *filter,
    int filter_is_f32, const void *direct, size_t length, size_t width,
    size_t groups, size_t taps, int orientation, void *pregate,
    float *inner_cache, float *short_cache, void *output, void *stream) {
  if (projection == nullptr)
    return fail(kInvalidArgument, "projection input is required");
  GatedFirArgs a;
  a.projection = projection;
  a.short_filter = short_filter;
  a.short_taps = 3;
  a.filter = filter;
  a.filter_is_f32 = filter_is_f32 != 0;
  a.direct = direct;
  a.length = length;
  a.width = width;
  a.groups = groups;
  a.taps = taps;
  a.cross_correlation = orientation == 0;
  a.pregate = pregate;
  a.inner_cache = inner_cache;
  a.short_cache = short_cache;
  a.output = output;
  return gated_fir_prefill(a, as_stream(stream));
}

size_t evo_b200_hcl_scratch_floats(size_t length, size_t width, size_t modes) {
  return modal_scratch_floats(length, width, modes);
}

int evo_b200_bf16_hcl_prefill(const void *x2, const void *x1, const void *value,
                              const void *direct, const float *log_poles,
                              const float *residues, size_t length,
                              size_t width, size_t modes, int mode,
                              float *state, float *scratch, void *pregate,
                              void *output, void *stream) {
  ModalArgs a;
  a.x2 = x2;
  a.x1 = x1;
  a.value = value;
  a.direct = direct;
  a.log_poles = log_poles;
  a.residues = residues;
  a.length = length;
  a.width = width;
  a.modes = modes;
  a.continue_from_state = mode == 1;
  a.state = state;
  a.scratch = scratch;
  a.pregate = pregate;
  a.output = output;
  return modal_prefill(a, as_stream(stream));
}

int evo_b200_bf16_hcl_prefill_noalloc(const void *x2, const void *x1, const void *value,
                                      const void *direct, const float *log_poles,
                                      const float *residues, size_t length, size_t width,
                                      size_t modes, int mode, float *state, void *pregate,
                                      void *output, void *stream) {
  ModalArgs a;
  a.x2 = x2;
  a.x1 = x1;
  a.value = value;
  a.direct = direct;
  a.log_poles = log_poles;
  a.residues = residues;
  a.length = length;
  a.width = width;
  a.modes = modes;
  a.continue_from_state = mode == 1;
  a.state = state;
  a.pregate = pregate;
  a.output = output;
  return modal_prefill_static_scratch(a, as_stream(stream));
}

int evo_b200_bf16_projection_hcl_prefill(
    const void *projection, const void *short_filter, const void *direct,
    const float *log_poles, const float *residues, size_t length, size_t width,
    size_t modes, int mode, float *state, float *scratch, float *short_cache,
    void *pregate, void *output, void *stream) {
  if (projection == nullptr)
    return fail(kInvalidArgument, "projection input is required");
  ModalArgs a;
  a.projection = projection;
  a.short_filter = short_filter;
  a.short_taps = 3;
  a.direct = direct;
  a.log_poles = log_poles;
  a.residues = residues;
  a.length = length;
  a.width = width;
  a.modes = modes;
  a.continue_from_state = mode == 1;
  a.state = state;
  a.scratch = scratch;
  a.short_cache = short_cache;
  a.pregate = pregate;
  a.output = output;
  return modal_prefill(a, as_stream(stream));
}

int evo_b200_bf16_hcl_decode(const void *x2, const void *x1, const void *value,
                             const void *direct, const float *log_poles,
                             const float *residues, size_t width, size_t modes,
                             float *state, void *pregate, void *output,
                             void *stream) {
  return modal_decode(x2, x1, value, direct, log_poles, residues, width, modes,
                      state, pregate, output, as_stream(stream));
}

int evo_b200_bf16_split_rope_append(const void *qkv,
                                    const float *inverse_frequency, size_t rows,
                                    size_t heads, size_t head_dim,
                                    size_t position_offset,
                                    float position_scale, int head_major,
                                    void *query, void *key_cache,
                                    void *value_cache, size_t cache_capacity,
                                    void *stream) {
  return split_rope_append(qkv, inverse_frequency, rows, heads, head_dim,
                           position_offset, position_scale, head_major != 0,
                           query, key_cache, value_cache, cache_capacity,
                           as_stream(stream));
}

int evo_b200_bf16_causal_attention(const void *query, const void *key_cache,
                                   const void *value_cache, size_t rows,
                                   size_t total_keys, size_t heads,
                                   size_t head_dim, void *output, void *stream) {
  return causal_attention(query, key_cache, value_cache, rows, total_keys,
                          heads, head_dim, output, as_stream(stream));
}

int evo_b200_bf16_causal_attention_mma_sync(const void *query, const void *key_cache,
                                            const void *value_cache, size_t rows,
                                            size_t total_keys, size_t heads,
                                            size_t head_dim, void *output, void *stream) {
  return causal_attention_mma_sync(query, key_cache, value_cache, rows, total_keys,
                                   heads, head_dim, output, as_stream(stream));
}

int evo_b200_bf16_cached_cross_attention(const void *query,
                                         const void *key_cache,
                                         const void *value_cache, size_t rows,
                                         size_t total_keys, size_t heads,
                                         size_t head_dim, void *output,
                                         void *stream) {
  return cached_attention(query, key_cache, value_cache, rows, total_keys,
                          heads, head_dim, output, as_stream(stream));
}

int evo_b200_bf16_cached_cross_attention_probabilities(const void *query, const void *key_cache,
                                                       const void *value_cache, size_t rows, size_t total_keys,
                                                       size_t heads, size_t head_dim, void *probabilities,
                                                       void *output, void *stream) {
  return cached_attention(query, key_cache, value_cache, rows, total_keys, heads, head_dim, output,
                          as_stream(stream), probabilities);
}

// ---- LinearExecutor offload (src/linear_executor.hpp:13-28)
int evo_b200_linear_executor_create(int device, evo_b200_linear_executor **executor_out) {
  return linear_executor_create(device, reinterpret_cast<LinearExecutorState **>(executor_out));
}
void evo_b200_linear_executor_free(evo_b200_linear_executor *executor) {
  linear_executor_free(reinterpret_cast<LinearExecutorState *>(executor));
}
const char *evo_b200_linear_executor_name(void) { return "b200-tcgen05-bf16x3"; }
size_t evo_b200_linear_executor_cached_bytes(evo_b200_linear_executor *executor) {
  return linear_executor_cached_bytes(reinterpret_cast<LinearExecutorState *>(executor));
}
int evo_b200_linear_executor_linear(evo_b200_linear_executor *executor, const float *input, size_t rows,
                                    size_t input_width, const void *weight, int weight_dtype,
                                    size_t weight_elements, size_t output_width, const void *bias,
                                    int bias_dtype, size_t bias_elements, float *output) {
  return linear_executor_linear(reinterpret_cast<LinearExecutorState *>(executor), input, rows, input_width,
                                weight, weight_dtype, weight_elements, output_width, bias, bias_dtype,
                                bias_elements, output);
}

// ---- quantised KV cache
static Q8PageTable q8_table(void *const *key_pages, void *const *value_pages, void *const *key_scale_pages,
                            void *const *value_scale_pages, size_t page_tokens) {
  Q8PageTable table;
  table.key = reinterpret_cast<std::int8_t *const *>(key_pages);
  table.value = reinterpret_cast<std::int8_t *const *>(value_pages);
  table.key_scale = reinterpret_cast<float *const *>(key_scale_pages);
  table.value_scale = reinterpret_cast<float *const *>(value_scale_pages);
  table.page_tokens = page_tokens;
  return table;
}
int evo_b200_q8_kv_append(const void *key, const void *value, void *const *key_pages, void *const *value_pages,
                          void *const *key_scale_pages, void *const *value_scale_pages, size_t page_tokens,
                          size_t first_position, size_t rows, size_t heads, size_t head_dim, void *stream) {
  return q8_kv_append(key, value, q8_table(key_pages, value_pages, key_scale_pages, value_scale_pages, page_tokens),
                      first_position, rows, heads, head_dim, as_stream(stream));
}
int evo_b200_q8_kv_expand(void *const *key_pages, void *const *value_pages, void *const *key_scale_pages,
                          void *const *value_scale_pages, size_t page_tokens, size_t count, size_t heads,
                          size_t head_dim, void *key, void *value, void *stream) {
  return q8_kv_expand(q8_table(key_pages, value_pages, key_scale_pages, value_scale_pages, page_tokens), count, heads,
                      head_dim, key, value, as_stream(stream));
}
int evo_b200_q8_attention_decode(const void *query, void *const *key_pages, void *const *value_pages,
                                 void *const *key_scale_pages, void *const *value_scale_pages, size_t page_tokens,
                                 size_t rows, size_t total_keys, size_t heads, size_t head_dim, void *output,
                                 void *stream) {
  return q8_attention_decode(query, q8_table(key_pages, value_pages, key_scale_pages, value_scale_pages, page_tokens),
                             rows, total_keys, heads, head_dim, output, as_stream(stream));
}

// ---- host E4M3FN codec (include/evo/fp8.hpp)
uint8_t evo_b200_e4m3_encode(float value) { return fp8::encode_e4m3fn(value); }
float evo_b200_e4m3_decode(uint8_t code) { return fp8::decode_e4m3fn(code); }
float evo_b200_e4m3_scaled_roundtrip(float value, float scale) {
  return fp8::scaled_e4m3fn_roundtrip(value, scale);
}
int evo_b200_e4m3_encode_array(const float *values, size_t count, float scale, uint8_t *codes) {
  if ((values == nullptr || codes == nullptr) && count != 0)
    return fail(kInvalidArgument, "E4M3 encode arguments are invalid");
  if (!fp8::valid_scale(scale)) return fail(kInvalidArgument, "E4M3 scale must be positive and finite");
  for (size_t i = 0; i < count; ++i) codes[i] = fp8::encode_e4m3fn(values[i] * scale);
  return kOk;
}

}  // extern "C"
