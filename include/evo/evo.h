/* Model-level C ABI of the B200 StripedHyena2 runtime.
 *
 * Binary-compatible with upstream evo.cpp's include/evo/evo.h (ABI 1.5.0,
 * lines 24-210 there): the same 39 symbols, enumerators, parameter-struct
 * layouts, callback types and ownership rules, so a program linked against
 * upstream's libevo.so.1 can load this library instead.  Behind it sits the
 * sm_100a runtime of this repository (CUDA backend only; no CPU fallback).
 *
 * Additions that do not change existing layouts: the context flags
 * EVO_CONTEXT_FLAG_B200_*, and the evo_b200_* extension entry
 * points declared separately in evo_b200.h (not part of upstream's ABI).
 */
#ifndef EVO_EVO_H
#define EVO_EVO_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define EVO_API __attribute__((visibility("default")))
#else
#define EVO_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define EVO_ABI_VERSION_MAJOR 1u
#define EVO_ABI_VERSION_MINOR 5u
#define EVO_ABI_VERSION_PATCH 0u
#define EVO_ABI_VERSION_ENCODE(major, minor, patch) \
  ((((uint32_t)(major)&0xffu) << 24u) | (((uint32_t)(minor)&0xffu) << 16u) | \
   ((uint32_t)(patch)&0xffffu))
#define EVO_ABI_VERSION_CURRENT \
  EVO_ABI_VERSION_ENCODE(EVO_ABI_VERSION_MAJOR, EVO_ABI_VERSION_MINOR, EVO_ABI_VERSION_PATCH)

/* evo.h:34-43 upstream */
typedef enum evo_status {
  EVO_STATUS_OK = 0,
  EVO_STATUS_INVALID_ARGUMENT = 2,
  EVO_STATUS_IO = 3,
  EVO_STATUS_MODEL_FORMAT = 4,
  EVO_STATUS_UNSUPPORTED = 5,
  EVO_STATUS_CUDA = 6,
  EVO_STATUS_MPS = 7,
  EVO_STATUS_INTERNAL = 70
} evo_status;

typedef enum evo_backend {
  EVO_BACKEND_AUTO = 0,
  EVO_BACKEND_CUDA = 1,
  EVO_BACKEND_CPU = 2,
  EVO_BACKEND_MPS = 3
} evo_backend;

enum { EVO_MODEL_FLAG_TEST_ONLY_ALLOW_SYNTHETIC = 1u << 0u };
enum {
  EVO_CONTEXT_FLAG_FAST_Q8_KV = 1u << 0u,
  /* E4M3 Hyena projections run on tcgen05 FP8 tensor cores (profile
   * "b200-tc") instead of the bit-exact software emulation ("exact"). */
  EVO_CONTEXT_FLAG_B200_TENSORCORE_FP8 = 1u << 8u,
  /* Test fixtures normally get upstream's 8-row activation arena; this flag
   * gives them the production arena (8192 rows) so that long single-chunk
   * prefills of small synthetic models can be tested. */
  EVO_CONTEXT_FLAG_B200_FULL_ARENA = 1u << 9u,
  /* Profile "b200-fp8": as "b200-tc", and in prefill chunks of more than 128
   * rows the output projection and the three MLP projections of every block
   * also run as E4M3 tcgen05 GEMMs - weights quantised once per model with a
   * per-tensor scale 448 / max|w|, activations quantised per row with
   * 448 / max|row| just before each product, F32 accumulation, the BF16
   * epilogues unchanged.  Upstream keeps these projections in BF16
   * (src/cuda/ops.cu:1205-1245, src/cuda/model.cu:1787-1791, 1823-1825), so
   * this is new arithmetic under its own name, with tolerance parity against
   * "exact" (upstream's rule for approximate profiles:
   * docs/execution-profiles.md:77-82).  Implies the tensor-core projections. */
  EVO_CONTEXT_FLAG_B200_FP8_FFN = 1u << 10u
};

typedef struct evo_model evo_model;
typedef struct evo_context evo_context;
typedef struct evo_batch evo_batch;
typedef struct evo_sampler evo_sampler;

typedef struct evo_model_params {
  size_t struct_size;
  evo_backend backend;
  const int32_t *devices; /* pipeline stages, one CUDA device each */
  size_t device_count;
  uint32_t flags;
} evo_model_params;

typedef struct evo_context_params {
  size_t struct_size;
  size_t context_size;
  uint32_t flags;
} evo_context_params;

typedef struct evo_sampler_params {
  size_t struct_size;
  float temperature;
  size_t top_k;
  float top_p;
  uint64_t seed;
} evo_sampler_params;

typedef struct evo_embedding_options {
  size_t struct_size;
  const char *preset;
  size_t layer;
  const char *pooling;
} evo_embedding_options;

typedef struct evo_embedding_result_info {
  size_t struct_size;
  const char *resolved_preset;
  const char *hidden_tap;
  const char *pooling;
  size_t layer;
  size_t original_length;
  size_t effective_length;
  size_t crop_left;
  size_t crop_right;
  size_t pad_left;
  size_t pad_right;
  size_t token_count;
  size_t rows;
  size_t columns;
} evo_embedding_result_info;

/* Views are valid only during the call; a non-OK return aborts the
 * operation and permanently invalidates the context. */
typedef evo_status (*evo_logits_callback)(const float *logits, size_t rows, size_t columns,
                                          size_t token_offset, void *user_data);
typedef evo_status (*evo_embedding_callback)(const float *embedding, size_t rows,
                                             size_t columns, size_t token_offset,
                                             void *user_data);
typedef evo_status (*evo_embedding_ex_callback)(const float *embedding, size_t rows,
                                                size_t columns, size_t token_offset,
                                                const evo_embedding_result_info *info,
                                                void *user_data);

EVO_API uint32_t evo_abi_version(void);
EVO_API const char *evo_version_string(void);
EVO_API const char *evo_status_name(evo_status status);
EVO_API const char *evo_backend_name(evo_backend backend);
/* Thread-local "<code_name>: <message>", valid until the next call on this thread. */
EVO_API const char *evo_last_error(void);

EVO_API evo_model_params evo_model_default_params(void);
EVO_API evo_context_params evo_context_default_params(void);
EVO_API evo_sampler_params evo_sampler_default_params(void);
EVO_API evo_embedding_options evo_embedding_default_options(void);

EVO_API evo_status evo_model_load(const char *path, const evo_model_params *params,
                                  evo_model **model_out);
EVO_API void evo_model_free(evo_model *model);
EVO_API evo_backend evo_model_backend(const evo_model *model);
EVO_API const char *evo_model_id(const evo_model *model);
EVO_API const char *evo_model_architecture(const evo_model *model);
EVO_API const char *evo_model_profile(const evo_model *model);
EVO_API size_t evo_model_vocab_size(const evo_model *model);
EVO_API size_t evo_model_max_context(const evo_model *model);
EVO_API size_t evo_model_embedding_width(const evo_model *model);
EVO_API size_t evo_model_layer_count(const evo_model *model);
EVO_API evo_status evo_model_encode(const evo_model *model, const uint8_t *sequence,
                                    size_t sequence_length, uint32_t *tokens,
                                    size_t token_capacity, size_t *token_count);
EVO_API evo_status evo_model_decode_token(const evo_model *model, uint32_t token,
                                          uint8_t *byte_out);

/* A context keeps the device weights alive; the model handle may be freed first. */
EVO_API evo_status evo_context_create(const evo_model *model, const evo_context_params *params,
                                      evo_context **context_out);
EVO_API void evo_context_free(evo_context *context);
EVO_API size_t evo_context_position(const evo_context *context);
EVO_API size_t evo_context_capacity(const evo_context *context);
EVO_API const char *evo_context_profile(const evo_context *context);
EVO_API evo_status evo_context_prefill(evo_context *context, const evo_batch *batch,
                                       evo_logits_callback callback, void *user_data);
EVO_API evo_status evo_context_decode(evo_context *context, uint32_t token,
                                      evo_logits_callback callback, void *user_data);
EVO_API evo_status evo_context_embed(evo_context *context, const evo_batch *batch, size_t layer,
                                     evo_embedding_callback callback, void *user_data);
EVO_API evo_status evo_context_embed_ex(evo_context *context, const evo_batch *batch,
                                        const evo_embedding_options *options,
                                        evo_embedding_ex_callback callback, void *user_data);

EVO_API evo_status evo_batch_create(size_t sequence_capacity, evo_batch **batch_out);
EVO_API void evo_batch_free(evo_batch *batch);
EVO_API void evo_batch_clear(evo_batch *batch);
EVO_API evo_status evo_batch_add_sequence(evo_batch *batch, const uint8_t *sequence,
                                          size_t sequence_length);
EVO_API size_t evo_batch_sequence_count(const evo_batch *batch);
EVO_API size_t evo_batch_token_count(const evo_batch *batch);

EVO_API evo_status evo_sampler_create(const evo_sampler_params *params,
                                      evo_sampler **sampler_out);
EVO_API void evo_sampler_free(evo_sampler *sampler);
EVO_API evo_status evo_sampler_sample(evo_sampler *sampler, const float *logits,
                                      size_t logits_count, uint32_t *token_out);

#ifdef __cplusplus
}
#endif
#endif
