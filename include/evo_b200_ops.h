/* Operator-level C ABI of the B200 StripedHyena2 hot path.
 *
 * Every entry point takes raw device pointers on the current CUDA device, a
 * cudaStream_t passed as void*, and plain sizes; it enqueues work on that
 * stream and returns an evo_status value (0 = OK, 2 invalid argument,
 * 5 unsupported, 6 CUDA).  evo_b200_last_error() returns the thread-local
 * "<code_name>: <message>" text of the most recent failure on this thread.
 * Buffers are BF16 unless stated otherwise.  Each declaration cites the
 * upstream evo.cpp operator (path:line in that project) whose contract it
 * implements; upstream's DeviceBuffer/Stream arguments become pointer + size.
 */
#ifndef EVO_B200_OPS_H
#define EVO_B200_OPS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define EVO_B200_API __attribute__((visibility("default")))
#else
#define EVO_B200_API
#endif

EVO_B200_API const char *evo_b200_last_error(void);
/* Synchronises the stream; non-zero if a tensor-core GEMM pipeline wait
 * timed out since the last check (the flag is cleared). */
EVO_B200_API int evo_b200_check_async_errors(void *stream);

/* include/evo/cuda/ops.hpp:81-103, src/cuda/ops.cu:232-275: E4M3FN RNE
 * satfinite codes of float(x)*scale; optional F32 dequantised copy. */
EVO_B200_API int evo_b200_software_e4m3_quantize_bf16(
    const void *input, size_t elements, float scale, void *codes_u8,
    float *dequantized_f32, void *stream);
EVO_B200_API int evo_b200_software_e4m3_quantize_f32_codes(
    const float *input, size_t elements, float scale, void *codes_u8,
    void *stream);

/* include/evo/cuda/ops.hpp:104-110, src/cuda/ops.cu:353-441,916-1006:
 * y = bf16(QGMMA_emulation(E4M3(x*input_scale), w_codes) * output_scale),
 * bit-exact integer emulation, K a multiple of 32.  codes_scratch holds
 * rows*in_features bytes. */
EVO_B200_API int evo_b200_software_e4m3_h100_linear(
    const void *input, const void *weight_codes, size_t rows,
    size_t in_features, size_t out_features, float input_scale,
    float output_scale, void *codes_scratch, void *output, void *stream);
/* Same operands on the tcgen05 FP8 tensor cores (F32 accumulation): the
 * tensor-core execution profile of the projection above. */
EVO_B200_API int evo_b200_e4m3_tensorcore_linear(
    const void *input, const void *weight_codes, size_t rows,
    size_t in_features, size_t out_features, float input_scale,
    float output_scale, void *codes_scratch, void *output, void *stream);

/* Dynamic per-row quantisation in front of an E4M3 product (profile
 * "b200-fp8"; no upstream counterpart - upstream quantises with one static
 * scale per tensor, src/cuda/ops.cu:250-262): codes[r,:] = E4M3(x[r,:] * q_r),
 * q_r = 448 / max|x[r,:]| (1 for a zero row), row_scale[r] = 1 / q_r (F32
 * [rows]).  width % 8 == 0, 16-byte aligned input. */
EVO_B200_API int evo_b200_e4m3_quantize_rows(const void *input, size_t rows, size_t width,
                                             void *codes_u8, float *row_scale, void *stream);
/* y = epilogue(alpha * row_scale[r] * (codes_x . codes_w^T)) on the tcgen05 FP8
 * tensor cores, F32 accumulation; bias / residual / gate as in
 * evo_b200_bf16_linear and evo_b200_bf16_gated_up_projection (gate_mode 0 none,
 * 1 product of the interleaved 128-column halves, 2 GELU on the first half;
 * a gated call takes no bias or residual and writes out_features / 2 columns).
 * row_scale may be NULL. */
EVO_B200_API int evo_b200_e4m3_codes_linear(const void *input_codes, const float *row_scale,
                                            const void *weight_codes, const void *bias,
                                            const void *residual, size_t rows, size_t in_features,
                                            size_t out_features, float alpha, int bias_mode,
                                            int gate_mode, void *output, void *stream);

/* include/evo/cuda/ops.hpp:37-68, src/cuda/ops.cu:535-748: y = x W^T with
 * W [out,in]; bias_mode 0 none, 1 fused into the F32 sum (cuBLASLt BIAS
 * epilogue upstream), 2 separate BF16-rounded add
 * (bf16_add_bias_inplace, src/cuda/ops.cu:187-198); residual (optional) is
 * added last with its own rounding (bf16_add_inplace, ops.cu:175-185).
 * path 0 = tcgen05 when the shape allows, 1 = CUDA-core kernel. */
EVO_B200_API int evo_b200_bf16_linear(const void *input, const void *weight,
                                      const void *bias, const void *residual,
                                      size_t rows, size_t in_features,
                                      size_t out_features, int bias_mode,
                                      int path, void *output, void *stream);
/* The same projection with scratch for split-K (no upstream counterpart:
 * cuBLASLt owns its workspace there).  At 9..128 rows a projection is a weight
 * stream with fewer output tiles than SMs; with a workspace the weights become
 * the 128-row tensor-core operand and the tokens the narrow one, the K
 * dimension is split over up to 8 CTAs per 128 weight rows, F32 partial sums
 * go to the workspace (split * rows * out_features floats are needed, less is
 * fine: fewer splits, or the one-pass kernel when not even one fits) and are
 * added in split order.  gate_mode 0 none, 1 / 2 = the gated
 * up-projection of evo_b200_bf16_gated_up_projection (identity / GELU) with
 * out_features = 2 * inner width.  The workspace must not be shared by calls
 * that may overlap on the GPU. */
EVO_B200_API int evo_b200_bf16_linear_split_k(
    const void *input, const void *weight, const void *bias,
    const void *residual, size_t rows, size_t in_features, size_t out_features,
    int bias_mode, int gate_mode, void *workspace, size_t workspace_bytes,
    void *output, void *stream);
/* src/cuda/ops.cu:1205-1245 (bf16_mlp first half): gated = act(x W1^T) *
 * (x W2^T) in one GEMM over a row-interleaved [W1 | W2] weight built by
 * evo_b200_interleave_gate_weights; activation 0 identity, 1 GELU. */
EVO_B200_API int evo_b200_bf16_gated_up_projection(
    const void *input, const void *interleaved_weight, size_t rows,
    size_t in_features, size_t inner_width, int activation, void *output,
    void *stream);
EVO_B200_API int evo_b200_interleave_gate_weights(const void *w1,
                                                  const void *w2,
                                                  size_t inner_width,
                                                  size_t in_features,
                                                  void *interleaved,
                                                  void *stream);

/* include/evo/cuda/ops.hpp:111-120, src/cuda/ops.cu:72-113.  output and
 * codes_u8 are each optional (at least one); codes = E4M3(y*quant_scale). */
EVO_B200_API int evo_b200_bf16_rms_norm(const void *input, const float *scale,
                                        size_t rows, size_t width,
                                        float epsilon, void *output,
                                        void *codes_u8, float quant_scale,
                                        void *stream);
/* include/evo/cuda/ops.hpp:121-135, src/cuda/ops.cu:115-198. */
EVO_B200_API int evo_b200_bf16_gelu(const void *input, size_t elements,
                                    void *output, void *stream);
EVO_B200_API int evo_b200_bf16_gated_elementwise(const void *first,
                                                 const void *second,
                                                 size_t elements, int gelu,
                                                 void *output, void *stream);
EVO_B200_API int evo_b200_bf16_add(const void *first, const void *second,
                                   size_t elements, void *output,
                                   void *stream);
EVO_B200_API int evo_b200_bf16_add_bias_inplace(void *output, const void *bias,
                                                size_t rows, size_t width,
                                                void *stream);
/* include/evo/cuda/ops.hpp:73-80, src/cuda/ops.cu:200-230. */
EVO_B200_API int evo_b200_bf16_row_to_column_major(const void *input,
                                                   size_t rows, size_t columns,
                                                   void *output, void *stream);
/* src/cuda/model.cu:269-284. tokens are uint32 ids on the device; `vocabulary`
 * is the number of table rows.  An id >= vocabulary is never used as an index:
 * its output row is zeros and the next evo_b200_check_async_errors on the
 * device returns invalid_argument (upstream validates ids on the host,
 * src/cuda/model.cu:1872-1880, before they reach the device). */
EVO_B200_API int evo_b200_embedding(const uint32_t *tokens, const void *table,
                                    size_t rows, size_t width, size_t vocabulary,
                                    void *output, void *stream);

/* include/evo/cuda/hyena.hpp (bf16_split_hyena_projection),
 * src/cuda/hyena.cu:194-208. */
EVO_B200_API int evo_b200_bf16_split_hyena_projection(
    const void *projection, size_t rows, size_t width, void *x2, void *x1,
    void *value, void *stream);
/* src/cuda/hyena.cu:243-272,1525-1581 (bf16_fir_prefill_direct).  filter is
 * [groups, taps] BF16 (filter_is_f32 = 0) or F32; orientation 0 =
 * cross-correlation, 1 = causal convolution; bias_mode 0 add, 1 multiply by
 * the input; cache (optional) receives the last taps-1 inputs as F32
 * [channels, taps-1]. */
EVO_B200_API int evo_b200_bf16_fir_prefill_direct(
    const void *input, const void *filter, int filter_is_f32, const void *bias,
    size_t length, size_t channels, size_t groups, size_t taps,
    int orientation, int bias_mode, void *output, float *cache, void *stream);
/* src/cuda/hyena.cu:275-416,1583-1652,1737-1790 (bf16_fir_continue_direct /
 * bf16_fir_decode): length >= 1 new rows against cache_length cached rows;
 * the cache is advanced afterwards. */
EVO_B200_API int evo_b200_bf16_fir_continue_direct(
    const void *input, const void *filter, int filter_is_f32, const void *bias,
    size_t length, size_t channels, size_t groups, size_t taps,
    int orientation, int bias_mode, float *cache, size_t cache_length,
    void *output, void *stream);
/* include/evo/cuda/hyena.hpp:203-250 (bf16_hcs_prefill, bf16_hcm_prefill,
 * bf16_hcm_prefill_direct): out = bf16(bf16(fir(bf16(x1*v)) [+ direct*u]) *
 * x2) in one fused pass.  direct may be NULL (HCS).  pregate (optional)
 * receives u; inner_cache (optional) the F32 tail of u.  An odd width runs
 * as three passes (gate, FIR, gate) and needs pregate. */
EVO_B200_API int evo_b200_bf16_gated_fir_prefill(
    const void *x2, const void *x1, const void *value, const void *filter,
    int filter_is_f32, const void *direct, size_t length, size_t width,
    size_t groups, size_t taps, int orientation, void *pregate,
    float *inner_cache, void *output, void *stream);
/* Row-window forms used by chunked prefill inside one activation arena
 * (upstream's continuation operators bf16_hcs_continue / bf16_hcm_continue /
 * HclPrefillMode::kRecurrenceContinue, include/evo/cuda/hyena.hpp:216-250, keep
 * the history in F32 caches instead): only rows [row_begin, length) are
 * produced; earlier rows of the same input buffers are the history.  For the
 * HCL form *state must hold the modal state after row_begin-1 (mode 1). */
EVO_B200_API int evo_b200_bf16_gated_fir_prefill_window(
    const void *x2, const void *x1, const void *value, const void *filter,
    int filter_is_f32, const void *direct, size_t row_begin, size_t length,
    size_t width, size_t groups, size_t taps, int orientation,
    float *inner_cache, void *output, void *stream);
EVO_B200_API int evo_b200_bf16_hcl_prefill_window(
    const void *x2, const void *x1, const void *value, const void *direct,
    const float *log_poles, const float *residues, size_t row_begin,
    size_t length, size_t width, size_t modes, float *state, float *scratch,
    void *output, void *stream);
/* The same operator fed by the raw interleaved projection [length, 3*width]
 * with the 3-tap featurizer [3*width, 3] applied on the fly
 * (src/cuda/model.cu:1431-1470 + 1477-1520 in one pass). */
EVO_B200_API int evo_b200_bf16_projection_gated_fir_prefill(
    const void *projection, const void *short_filter, const void *filter,
    int filter_is_f32, const void *direct, size_t length, size_t width,
    size_t groups, size_t taps, int orientation, void *pregate,
    float *inner_cache, float *short_cache, void *output, void *stream);

/* include/evo/cuda/hyena.hpp (bf16_hcl_prefill), src/cuda/hyena.cu:1994-2124.
 * mode 0: initial prefill (state written if non-NULL, four BF16 roundings),
 * mode 1: continuation from *state (single rounding).  scratch must hold
 * evo_b200_hcl_scratch_floats(length,width,modes) floats. */
EVO_B200_API size_t evo_b200_hcl_scratch_floats(size_t length, size_t width,
                                                size_t modes);
EVO_B200_API int evo_b200_bf16_hcl_prefill(
    const void *x2, const void *x1, const void *value, const void *direct,
    const float *log_poles, const float *residues, size_t length, size_t width,
    size_t modes, int mode, float *state, float *scratch, void *pregate,
    void *output, void *stream);
/* No counterpart in upstream evo.cpp.  evo_b200_bf16_hcl_prefill for callers
 * that must not touch the CUDA allocator: a serving process that handed all
 * free device memory to its own pool at start-up (so a later cudaMalloc fails
 * or fragments it), or a latency-critical loop that cannot afford the implicit
 * device synchronisation of cudaMalloc/cudaFree.  Inputs, outputs and state
 * are still the caller's buffers; only the segment-state scratch differs: it
 * is a fixed 4 Mi-float (16 MiB) array inside the library image, resident on
 * every GPU that loads the library until the process exits.
 *  - Limit: one state of width * modes floats per row segment plus one must
 *    fit the array; fewer, longer segments are used when they do not, so the
 *    call is refused (status 2, message names the limit) only when width *
 *    modes itself exceeds 4 Mi floats.
 *  - The first call on each device resolves the array's device address
 *    (cudaGetSymbolAddress, with that device current); make that first call
 *    outside any stream capture.
 *  - All calls on a device share the array.  Every call overwrites the part it
 *    uses before reading it, so nothing has to be cleared between calls, but
 *    two calls whose kernels overlap on the GPU (different streams) race.
 *  - The call itself performs no cudaMalloc, cudaFree or other allocating
 *    library call. */
EVO_B200_API int evo_b200_bf16_hcl_prefill_noalloc(
    const void *x2, const void *x1, const void *value, const void *direct,
    const float *log_poles, const float *residues, size_t length, size_t width,
    size_t modes, int mode, float *state, void *pregate, void *output,
    void *stream);
EVO_B200_API int evo_b200_bf16_projection_hcl_prefill(
    const void *projection, const void *short_filter, const void *direct,
    const float *log_poles, const float *residues, size_t length, size_t width,
    size_t modes, int mode, float *state, float *scratch, float *short_cache,
    void *pregate, void *output, void *stream);
/* One cached-decode step of a whole Hyena mixer in one launch (no upstream
 * counterpart: upstream runs the featurizer step, split, gate, bf16_fir_decode
 * or bf16_hcl_decode and the post-gate as separate launches,
 * src/cuda/model.cu:1471-1560).  Bit-identical to that sequence.  projection is
 * the token's [3 width] input projection; short_cache [3 width, 2], inner_cache
 * [width, taps-1] and modal_state [width, modes] are advanced in place and must
 * hold full histories.  FIR form: filter set, log_poles NULL (direct optional);
 * modal form: log_poles, residues, direct and modal_state set. */
EVO_B200_API int evo_b200_bf16_hyena_decode_mixer(
    const void *projection, const void *short_filter, float *short_cache,
    const void *direct, const void *filter, int filter_is_f32, size_t groups,
    size_t taps, int orientation, float *inner_cache, const float *log_poles,
    const float *residues, size_t modes, float *modal_state, size_t width,
    void *output, void *stream);
/* src/cuda/hyena.cu:718-761,2126-2167 (bf16_hcl_decode). */
EVO_B200_API int evo_b200_bf16_hcl_decode(
    const void *x2, const void *x1, const void *value, const void *direct,
    const float *log_poles, const float *residues, size_t width, size_t modes,
    float *state, void *pregate, void *output, void *stream);

/* include/evo/cuda/attention.hpp:92-140.  split + RoPE + KV append in one
 * pass (bf16_split_qkv, bf16_apply_rope, bf16_kv_append;
 * src/cuda/attention.cu:210-281): qkv [rows, 3*heads*head_dim]; caches are
 * [capacity, heads, head_dim] and rows are written at position_offset. */
EVO_B200_API int evo_b200_bf16_split_rope_append(
    const void *qkv, const float *inverse_frequency, size_t rows, size_t heads,
    size_t head_dim, size_t position_offset, float position_scale,
    int head_major, void *query, void *key_cache, void *value_cache,
    size_t cache_capacity, void *stream);
/* bf16_flash_causal_attention / bf16_online_causal_attention
 * (src/cuda/flash_attention.cu:199-441, src/cuda/attention.cu:879-1070). */
EVO_B200_API int evo_b200_bf16_causal_attention(
    const void *query, const void *key_cache, const void *value_cache,
    size_t rows, size_t total_keys, size_t heads, size_t head_dim,
    void *output, void *stream);
/* Same contract on warp-level MMAs (head size 128, >= 16 rows) or the row-wise
 * kernel: what evo_b200_bf16_causal_attention uses below 128 rows and for
 * other head sizes; exported as a cross-check of the tcgen05 kernel. */
EVO_B200_API int evo_b200_bf16_causal_attention_mma_sync(
    const void *query, const void *key_cache, const void *value_cache,
    size_t rows, size_t total_keys, size_t heads, size_t head_dim,
    void *output, void *stream);
/* bf16_cached_cross_attention (src/cuda/attention.cu:283-784,1669-1799). */
EVO_B200_API int evo_b200_bf16_cached_cross_attention(
    const void *query, const void *key_cache, const void *value_cache,
    size_t rows, size_t total_keys, size_t heads, size_t head_dim,
    void *output, void *stream);
/* The same operator, also writing the BF16 probabilities [heads, rows,
 * total_keys] (zeros behind the causal boundary) that upstream materialises
 * between its two GEMMs (the `probabilities` scratch of
 * bf16_cached_cross_attention, include/evo/cuda/attention.hpp:131-140).
 * probabilities may be NULL. */
EVO_B200_API int evo_b200_bf16_cached_cross_attention_probabilities(
    const void *query, const void *key_cache, const void *value_cache,
    size_t rows, size_t total_keys, size_t heads, size_t head_dim,
    void *probabilities, void *output, void *stream);

/* ---- Dense-linear offload with the contract of upstream's LinearExecutor
 * (src/linear_executor.hpp:13-28; called from cpu::linear,
 * src/cpu/model.cpp:284-302): F32 host activations [rows, input_width], a host
 * weight [output_width, input_width] row-major (dtype 0 = F32, 1 = BF16, 2 = raw
 * E4M3 codes decoded without a scale as upstream's Metal executor does,
 * src/mps/model.mm:42-58: upstream TensorDType kF32 / kBF16 / kE4M3Software),
 * optional bias (dtype 0 or 1), F32 host output
 * [rows, output_width].  Operands are split into BF16 planes (exact to 2^-24)
 * and multiplied on the tensor cores; their accumulator truncates, so results
 * agree with F32 arithmetic to a few 1e-6 of sum(|x||w|).  Device copies of weights are cached by
 * host address for the executor's lifetime (as upstream's Metal executor does,
 * src/mps/model.mm:218-238), so the mapped model file must outlive it; calls
 * are serialised internally and return when the output is written.  Outputs
 * narrower than 64 columns are refused with status 5 (keep them on the host).
 * There is one stream and one weight cache per executor; create one executor
 * per GPU. */
typedef struct evo_b200_linear_executor evo_b200_linear_executor;
EVO_B200_API int evo_b200_linear_executor_create(int device, evo_b200_linear_executor **executor_out);
EVO_B200_API void evo_b200_linear_executor_free(evo_b200_linear_executor *executor);
EVO_B200_API const char *evo_b200_linear_executor_name(void);
EVO_B200_API size_t evo_b200_linear_executor_cached_bytes(evo_b200_linear_executor *executor);
EVO_B200_API int evo_b200_linear_executor_linear(
    evo_b200_linear_executor *executor, const float *input, size_t rows,
    size_t input_width, const void *weight, int weight_dtype,
    size_t weight_elements, size_t output_width, const void *bias,
    int bias_dtype, size_t bias_elements, float *output);


/* ---- quantised KV cache (profile fast-q8-kv; upstream src/cuda/attention.cu:798-866 append,
 * :1072-1141 attention; docs/execution-profiles.md:96-127).  A cache is four device arrays of
 * page pointers - key codes, value codes (int8 [page_tokens, heads, head_dim]) and key scales, value
 * scales (F32 [page_tokens, heads]); page p holds positions [p * page_tokens, (p+1) * page_tokens).
 * Every (token, head) vector has scale = max|v| / 127 (1 for a zero vector) and codes
 * clamp(rint(v / scale), -127, 127).  append quantises BF16 K / V [rows, heads, head_dim] of positions
 * first_position ..; expand writes BF16 images [count, heads, head_dim] of positions [0, count);
 * attention_decode is causal attention of 1..8 query rows (row i sees keys 0 .. total_keys - rows
 * + i) read straight from the pages, head size 128 only (append and expand take any head size). */
EVO_B200_API int evo_b200_q8_kv_append(const void *key, const void *value, void *const *key_pages,
                                       void *const *value_pages, void *const *key_scale_pages,
                                       void *const *value_scale_pages, size_t page_tokens,
                                       size_t first_position, size_t rows, size_t heads, size_t head_dim,
                                       void *stream);
EVO_B200_API int evo_b200_q8_kv_expand(void *const *key_pages, void *const *value_pages,
                                       void *const *key_scale_pages, void *const *value_scale_pages,
                                       size_t page_tokens, size_t count, size_t heads, size_t head_dim,
                                       void *key, void *value, void *stream);
EVO_B200_API int evo_b200_q8_attention_decode(const void *query, void *const *key_pages,
                                              void *const *value_pages, void *const *key_scale_pages,
                                              void *const *value_scale_pages, size_t page_tokens, size_t rows,
                                              size_t total_keys, size_t heads, size_t head_dim, void *output,
                                              void *stream);

/* ---- host E4M3FN codec (no GPU needed): upstream evo::fp8
 * (include/evo/fp8.hpp:9-18, src/fp8.cpp:26-77).  Round-to-nearest-even,
 * satfinite (|v| >= 448 and infinities -> +-448), NaN -> 0x7f | sign.
 * evo_b200_e4m3_scaled_roundtrip = decode(encode(value * scale)) * (1 / scale),
 * NaN for a scale that is not positive and finite.  The array form encodes
 * `count` values times `scale`. */
EVO_B200_API uint8_t evo_b200_e4m3_encode(float value);
EVO_B200_API float evo_b200_e4m3_decode(uint8_t code);
EVO_B200_API float evo_b200_e4m3_scaled_roundtrip(float value, float scale);
EVO_B200_API int evo_b200_e4m3_encode_array(const float *values, size_t count, float scale,
                                            uint8_t *codes);

#ifdef __cplusplus
}
#endif
#endif
