/* Extension entry points of the B200 runtime.  They have no counterpart in
 * upstream evo.cpp's C ABI; they expose what a benchmark or a multi-process
 * launcher needs beyond it: device-resident token input, the context's CUDA
 * stream for event timing, and the stage layout of the layer pipeline
 * (upstream reports the latter through StageAssignment,
 * include/evo/cuda/model.hpp:94-101, which its C ABI does not export). */
#ifndef EVO_EVO_B200_H
#define EVO_EVO_B200_H

#include "evo.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct evo_b200_stage_info {
  size_t struct_size;
  int32_t device;
  size_t layer_begin;
  size_t layer_end;
  size_t weight_bytes;
  size_t cache_bytes;
  size_t arena_bytes;
} evo_b200_stage_info;

/* Enqueues one prefill of `rows` token ids that already live on the device of
 * pipeline stage 0 (uint32, rows <= activation capacity) on the context's
 * stream and returns without waiting.  BF16 logits [rows, vocab] stay on the
 * device; *device_logits_out (optional) receives their address.  stateless != 0
 * keeps no caches (position stays 0); otherwise the context is left ready for
 * decode.  Call evo_b200_context_synchronize before reading results. */
EVO_API evo_status evo_b200_context_prefill_device(evo_context *context,
                                                   const uint32_t *device_tokens, size_t rows,
                                                   int stateless,
                                                   const void **device_logits_out);
/* The next `rows` tokens of the same sequence (after a non-stateless prefill or
 * an earlier continuation): same conventions as evo_b200_context_prefill_device.
 * This is what evo_context_prefill does for every chunk after the first when a
 * prompt is longer than the activation capacity (upstream:
 * PipelineModel::prefill_chunk, include/evo/cuda/model.hpp:150-170). */
EVO_API evo_status evo_b200_context_continue_device(evo_context *context,
                                                    const uint32_t *device_tokens, size_t rows,
                                                    const void **device_logits_out);
/* The prefill forms of upstream's model classes that the portable ABI folds into evo_context_prefill
 * (SingleGpuModel / PipelineModel, include/evo/cuda/model.hpp:121-170), on token ids instead of bytes:
 *   FRESH      prefill(): starts a new sequence on any context (earlier state is dropped); prompts
 *              longer than the activation capacity run as chunks;
 *   STATELESS  prefill_stateless(): the same logits, no caches kept, position stays 0;
 *   CACHED     prefill_cached(): the exact cached-generation arithmetic (BF16 score and probability
 *              tensors); continues through evo_context_decode only;
 *   CHUNK      prefill_chunk(): the next tokens of the sequence a FRESH prefill started.
 * STATELESS, CACHED and CHUNK take at most evo_b200_context_activation_capacity tokens.  The
 * callback receives the rows of each chunk as evo_context_prefill delivers them. */
enum {
  EVO_B200_PREFILL_FRESH = 0, EVO_B200_PREFILL_STATELESS = 1, EVO_B200_PREFILL_CACHED = 2,
  EVO_B200_PREFILL_CHUNK = 3
};
EVO_API evo_status evo_b200_context_prefill_tokens(evo_context *context, const uint32_t *tokens,
                                                   size_t token_count, int32_t mode,
                                                   evo_logits_callback callback, void *user_data);
/* Block output of `layer` for one activation chunk of token ids (upstream prefill_embedding /
 * prefill_chunk_embedding, include/evo/cuda/model.hpp:150-170): first_chunk != 0 starts a new sequence
 * on any context, 0 continues the one a first chunk or a FRESH prefill started.  The context advances
 * as by a prefill; the callback receives [token_count, width] and the position of the first row. */
EVO_API evo_status evo_b200_context_embed_tokens(evo_context *context, const uint32_t *tokens,
                                                 size_t token_count, size_t layer, int32_t first_chunk,
                                                 evo_embedding_callback callback, void *user_data);
/* Rows of one activation chunk (upstream activation_capacity(), include/evo/cuda/model.hpp:141, 222). */
EVO_API size_t evo_b200_context_activation_capacity(const evo_context *context);
/* The runtime configuration of a model file without loading its weights (upstream
 * read_runtime_model_config + RuntimeModelConfig, include/evo/cuda/model.hpp:47-104): the same keys,
 * the same refusals (a synthetic fixture needs allow_test_fixture; precision metadata that disagrees
 * with the configuration, an unsupported projection dtype and tensors outside the profile's exact set
 * are rejected here, before any device work).  mixer_types (optional) receives one code per block -
 * 0 HCS, 1 HCM, 2 HCL, 3 attention - up to mixer_capacity.  The three names are NUL-terminated and cut
 * at 63 bytes. */
typedef struct evo_b200_model_config {
  size_t struct_size;
  char model_id[64];
  char architecture[64];
  char artifact_profile[64];
  size_t vocab_size, width, layers, heads, state_size, inner_width;
  size_t short_filter_length, hcs_filter_length, hcm_filter_length;
  size_t hcs_filter_groups, hcm_filter_groups, max_seqlen;
  float epsilon, rope_scale, rope_base;
  int32_t qkv_source_head_major;
  int32_t hyena_projection_e4m3; /* 0: BF16 projections, 1: E4M3 codes + software QGMMA contract */
  int32_t hcm_filter_f32;
  int32_t test_fixture;
} evo_b200_model_config;
EVO_API evo_status evo_b200_read_model_config(const char *path, int32_t allow_test_fixture,
                                              evo_b200_model_config *config, uint8_t *mixer_types,
                                              size_t mixer_capacity);
/* cudaStream_t of pipeline stage 0 (where a forward pass starts and ends). */
EVO_API void *evo_b200_context_stream(const evo_context *context);
/* Waits for all stages and reports asynchronous kernel errors. */
EVO_API evo_status evo_b200_context_synchronize(evo_context *context);
/* Per-operator timing: while enabled every operator launch is bracketed with
 * CUDA events on its stage stream (a few microseconds each, so leave it off for
 * throughput runs).  Enabling clears the totals.  evo_b200_context_profile_read
 * fills up to `capacity` entries with the milliseconds and launch counts per
 * operator class accumulated up to the last synchronising call and returns the
 * number of classes; evo_b200_profile_category_name names class `index`. */
EVO_API evo_status evo_b200_context_profile_enable(evo_context *context, int enabled);
EVO_API size_t evo_b200_context_profile_read(const evo_context *context, double *milliseconds,
                                             uint64_t *launches, size_t capacity);
EVO_API const char *evo_b200_profile_category_name(size_t index);
/* Host-only: the contiguous pipeline split used at load time.  layer_bytes[i] is
 * the tensor payload of block i; even_split != 0 selects the equal-count split
 * used for test fixtures.  Writes `stages` [begin, end) pairs; needs no GPU.
 * (Upstream computes the same split inside PipelineModel::load,
 * src/cuda/model.cu:2419-2469.) */
EVO_API evo_status evo_b200_plan_stages(const size_t *layer_bytes, size_t layers, size_t stages,
                                        int even_split, size_t *begins, size_t *ends);
EVO_API size_t evo_b200_context_stage_count(const evo_context *context);
EVO_API evo_status evo_b200_context_stage_info(const evo_context *context, size_t index,
                                               evo_b200_stage_info *info);


/* ---- activation taps inside the blocks.
 * Upstream's C++ runtime can write named intermediate activations of chosen
 * blocks to NPY files (LayerDumpPoint / LayerDump, include/evo/cuda/model.hpp:22-92;
 * PipelineModel::prefill_with_dumps, prefill_cached_with_dumps and
 * decode_with_dumps, :121-134 and :184-190; taken at src/cuda/model.cu:1373-1581
 * and :1757-1856); its C ABI does not export them.  Here they are a callback:
 * `point` is one of the 22 taps below, in upstream's order; values are F32
 * (BF16 activations widened; FIR histories and modal states are F32 already),
 * row-major [rows, columns], valid during the call.  Shapes: activations are
 * [tokens, width], [tokens, 3 width] for the projection and its featurizer
 * output, [tokens, inner] inside the MLP; mixer_short_state [3 width, filled
 * history], mixer_inner_state [width, filled history], mixer_state [width,
 * modes]; mixer_filter and mixer_convolution [tokens, width] (initial prefill of
 * a long-implicit block only).  Taps that a fused kernel keeps in registers are
 * produced by running the unfused operators for that block as well, so asking
 * for them costs extra launches; the block's results are unchanged.
 * The pass itself behaves like upstream's prefill_with_dumps (it starts a new
 * sequence on any context; one sequence, which must fit one activation chunk:
 * EVO_STATUS_UNSUPPORTED otherwise) and like evo_context_decode.  A non-OK status from either callback
 * aborts the pass and invalidates the context. */
enum {
  EVO_B200_DUMP_BLOCK_OUTPUT = 0, EVO_B200_DUMP_PRE_NORM, EVO_B200_DUMP_MIXER_INPUT_PROJECTION,
  EVO_B200_DUMP_MIXER_SHORT_FILTER, EVO_B200_DUMP_MIXER_SHORT_STATE, EVO_B200_DUMP_MIXER_INNER_STATE,
  EVO_B200_DUMP_MIXER_X2, EVO_B200_DUMP_MIXER_X1, EVO_B200_DUMP_MIXER_VALUE, EVO_B200_DUMP_MIXER_PREGATE,
  EVO_B200_DUMP_MIXER_STATE, EVO_B200_DUMP_MIXER_FILTER, EVO_B200_DUMP_MIXER_CONVOLUTION,
  EVO_B200_DUMP_MIXER_OUTPUT, EVO_B200_DUMP_MIXER_PROJECTION, EVO_B200_DUMP_MIXER_RESIDUAL,
  EVO_B200_DUMP_POST_NORM, EVO_B200_DUMP_MLP_L1, EVO_B200_DUMP_MLP_L2, EVO_B200_DUMP_MLP_ACTIVATION,
  EVO_B200_DUMP_MLP_GATED, EVO_B200_DUMP_MLP_OUTPUT, EVO_B200_DUMP_POINT_COUNT
};
typedef struct evo_b200_dump_request {
  size_t layer;
  int32_t point;
} evo_b200_dump_request;
typedef evo_status (*evo_b200_dump_callback)(size_t layer, int32_t point, const float *values,
                                             size_t rows, size_t columns, void *user_data);
/* "block_output", "pre_norm", "mixer_input_projection", ...: the file-name suffixes of
 * upstream's probe tool (tools/cuda_model_probe.cu:123-151); "" when out of range. */
EVO_API const char *evo_b200_dump_point_name(int32_t point);
EVO_API evo_status evo_b200_context_prefill_with_dumps(evo_context *context, const evo_batch *batch,
                                                       const evo_b200_dump_request *requests,
                                                       size_t request_count, int cached_attention,
                                                       evo_b200_dump_callback dump_callback,
                                                       evo_logits_callback logits_callback,
                                                       void *user_data);
EVO_API evo_status evo_b200_context_decode_with_dumps(evo_context *context, uint32_t token,
                                                      const evo_b200_dump_request *requests,
                                                      size_t request_count,
                                                      evo_b200_dump_callback dump_callback,
                                                      evo_logits_callback logits_callback,
                                                      void *user_data);

/* ---- variant-effect windows (host-only; need no GPU).
 * The sequence logic of upstream's `evo variant-score` driver
 * (src/variant.cpp:69-174, called from src/cuda/inference_cli.cpp:801-815):
 * the allele at 1-based `position` of `sequence` must equal `reference`; the
 * window keeps the allele and as much flank as `maximum_tokens` allows, half
 * on each side, a side that runs out of sequence ceding its share to the other.
 * `reference_window` / `alternate_window` receive the window with either allele
 * in place (capacity `window_capacity` bytes each, no terminator); all
 * sequences are IUPAC DNA, case kept.  EVO_STATUS_INVALID_ARGUMENT with
 * evo_last_error() set on a mismatch, a non-IUPAC byte, or a window that cannot
 * hold both alleles and two tokens. */
typedef struct evo_b200_variant_window {
  size_t struct_size;
  size_t reference_start; /* 0-based half-open span of the window on `sequence` */
  size_t reference_end;
  size_t variant_offset;  /* offset of the allele inside either window */
  size_t reference_length;
  size_t alternate_length;
} evo_b200_variant_window;
EVO_API evo_status evo_b200_variant_window_make(const char *sequence, size_t sequence_length,
                                                size_t position_1based, const char *reference,
                                                size_t reference_length, const char *alternate,
                                                size_t alternate_length, size_t maximum_tokens,
                                                evo_b200_variant_window *window, char *reference_window,
                                                char *alternate_window, size_t window_capacity);
/* Reverse complement of IUPAC DNA (upstream src/variant.cpp:86-101); `output` holds `length` bytes. */
EVO_API evo_status evo_b200_reverse_complement(const char *sequence, size_t length, char *output);

/* ---- file inputs of `evo variant-score --vcf ... --reference ...` (host-only).
 * Upstream: stream_vcf_file and fetch_reference_slice
 * (include/evo/variant_io.hpp:13-45, src/variant_io.cpp), driven from
 * src/cuda/inference_cli.cpp:939-975.  evo_b200_vcf_stream calls back once per
 * ALT allele of every record of a plain or gzip VCF ("-" = standard input);
 * the record's strings are valid during the call; a non-OK return stops the
 * stream and is returned.  evo_b200_reference_open scans a plain reference
 * FASTA once into an index (what a .fai holds; upstream re-reads the file twice
 * per allele instead), and evo_b200_reference_window checks that the contig
 * holds `reference` at the 1-based position and cuts the scoring window: as
 * much flank as `maximum_tokens` allows, half on each side, a side that runs
 * out of contig ceding its share to the other.  `sequence` (capacity bytes, no
 * terminator) receives bases [*start, *end) of the contig. */
typedef struct evo_b200_vcf_record {
  size_t struct_size;
  const char *contig;
  const char *id;
  const char *reference;
  const char *alternate;
  size_t position_1based;
  size_t record_index;
  size_t allele_index;
  size_t line_number;
} evo_b200_vcf_record;
typedef evo_status (*evo_b200_vcf_callback)(const evo_b200_vcf_record *record, void *user_data);
EVO_API evo_status evo_b200_vcf_stream(const char *path, evo_b200_vcf_callback callback, void *user_data);
typedef struct evo_b200_reference evo_b200_reference;
EVO_API evo_status evo_b200_reference_open(const char *path, evo_b200_reference **reference_out);
EVO_API void evo_b200_reference_free(evo_b200_reference *reference);
EVO_API evo_status evo_b200_reference_window(const evo_b200_reference *reference, const char *contig,
                                             size_t position_1based, const char *reference_allele,
                                             size_t reference_length, const char *alternate_allele,
                                             size_t alternate_length, size_t maximum_tokens,
                                             size_t *start, size_t *end, size_t *contig_length,
                                             char *sequence, size_t capacity);

/* ---- request scheduler over shared-weight contexts.
 * The serving loop behind upstream's `evo serve` (DynamicScheduler,
 * include/evo/server.hpp:59-88, src/scheduler.cpp:49-201; contexts that share
 * one copy of the weights, src/cuda/model.cu:2596-2691), without upstream's
 * HTTP transport (src/server.cpp), which is not part of this library.
 * `workers` threads each own one long-lived context of `context_size` tokens
 * and take requests from a bounded queue as they become free; upstream instead
 * runs batches of up to --max-batch requests behind a barrier and builds a
 * context per request.  A request is one sequence to score (sum and per-token
 * next-token log-likelihoods, the rule of `evo score`) or one prompt to extend
 * by new_tokens sampled tokens.
 *  - evo_b200_scheduler_submit copies the request, sets *ticket (0 when the
 *    queue is full: the request is refused and counted as rejected, status
 *    stays EVO_STATUS_OK) and returns at once; `done` runs later on a worker
 *    thread with the result, whose pointers are valid during the call.
 *  - evo_b200_scheduler_cancel marks a queued or running request: it completes
 *    with cancelled != 0 at its next check (before it starts, between prefill
 *    chunks, between decoded tokens).
 *  - evo_b200_scheduler_free cancels what is still queued, lets running
 *    requests reach their next check, and joins the workers; the model may be
 *    freed before or after. */
typedef struct evo_b200_scheduler evo_b200_scheduler;
typedef struct evo_b200_scheduler_params {
  size_t struct_size;
  size_t workers;        /* concurrent contexts, 1..64 */
  size_t maximum_queue;  /* >= workers */
  size_t context_size;   /* tokens per context */
  uint32_t context_flags; /* EVO_CONTEXT_FLAG_* of every context */
} evo_b200_scheduler_params;
enum { EVO_B200_REQUEST_SCORE = 0, EVO_B200_REQUEST_GENERATE = 1 };
typedef struct evo_b200_request {
  size_t struct_size;
  int32_t kind;
  const uint8_t *sequence;
  size_t length;
  size_t new_tokens;          /* generate only */
  evo_sampler_params sampler; /* generate only */
} evo_b200_request;
typedef struct evo_b200_request_result {
  size_t struct_size;
  evo_status status;
  const char *error; /* "" when status is OK */
  int32_t cancelled;
  double log_likelihood;
  size_t scored_tokens;
  const double *token_log_likelihoods; /* scored_tokens values */
  const uint8_t *generated;
  size_t generated_length;
  double queue_seconds;
  double run_seconds;
} evo_b200_request_result;
typedef void (*evo_b200_request_callback)(uint64_t ticket, const evo_b200_request_result *result,
                                          void *user_data);
typedef struct evo_b200_scheduler_metrics {
  size_t struct_size;
  uint64_t submitted, rejected, completed, failed, cancelled;
  size_t queued, queue_peak, active, active_peak;
} evo_b200_scheduler_metrics;
EVO_API evo_status evo_b200_scheduler_create(const evo_model *model, const evo_b200_scheduler_params *params,
                                             evo_b200_scheduler **scheduler_out);
EVO_API void evo_b200_scheduler_free(evo_b200_scheduler *scheduler);
EVO_API evo_status evo_b200_scheduler_submit(evo_b200_scheduler *scheduler, const evo_b200_request *request,
                                             evo_b200_request_callback done, void *user_data, uint64_t *ticket);
EVO_API int evo_b200_scheduler_cancel(evo_b200_scheduler *scheduler, uint64_t ticket);
EVO_API evo_status evo_b200_scheduler_read_metrics(const evo_b200_scheduler *scheduler,
                                                   evo_b200_scheduler_metrics *metrics);
EVO_API void evo_b200_scheduler_wait_idle(const evo_b200_scheduler *scheduler);

/* ---- one pipeline stage per process (torchrun / MPI style launchers).
 * Upstream runs its layer pipeline inside one process
 * (src/cuda/model.cu:2419-2469 plans the stages, :3148-3212 hands the hidden
 * rows from device to device); these calls expose one stage of the same plan
 * so that each process owns one GPU and the launcher moves the hidden rows
 * (NCCL send/recv or any peer copy) between them.
 *
 * evo_b200_model_load_slice loads stage `slice_index` of the `slice_count`-way
 * split of the artifact onto `device` (the first slice also holds the
 * embedding, the last slice the tied head and final norm).  A context of such a
 * model serves windowed prefills only: whole-model calls are refused.
 *
 * Per window of `rows` tokens starting at sequence position `position`, in
 * ascending contiguous order starting at 0, all enqueued on
 * evo_b200_context_stream():
 *   first slice:  slice_embed(tokens) -> slice_run -> send hidden rows
 *   middle:       receive hidden rows -> slice_run -> send hidden rows
 *   last slice:   receive hidden rows -> slice_run -> slice_head, which leaves
 *                 the window's BF16 logits on the device.
 * Position p lives at row p % capacity of evo_b200_context_slice_hidden (a
 * [capacity, width] BF16 buffer, capacity = the context's activation rows) and
 * of the logits buffer; a window may not straddle the end of that buffer, so
 * prompts longer than the capacity use windows that divide it.  State (KV
 * caches, FIR histories, modal states) is carried from window to window.
 * slice_embed's device_tokens points at the ids of the window (rows uint32). */
EVO_API evo_status evo_b200_model_load_slice(const char *path, int32_t device, size_t slice_index,
                                             size_t slice_count, uint32_t flags,
                                             evo_model **model_out);
EVO_API evo_status evo_b200_context_slice_embed(evo_context *context,
                                                const uint32_t *device_tokens, size_t position,
                                                size_t rows);
EVO_API evo_status evo_b200_context_slice_run(evo_context *context, size_t position, size_t rows);
/* *device_logits_out: start of the logits buffer (row = position % capacity). */
EVO_API evo_status evo_b200_context_slice_head(evo_context *context, size_t position, size_t rows,
                                               const void **device_logits_out);
EVO_API void *evo_b200_context_slice_hidden(const evo_context *context);

#ifdef __cplusplus
}
#endif
#endif
