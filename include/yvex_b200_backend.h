/*
 * yvex_b200 host boundary (C11): the slice of libyvex's backend operator surface that the
 * quantized MoE execution path crosses, re-implemented over the sm_100a device layer
 * (yvex_b200_kernels.h). Names, argument meaning, ownership rules and error behaviour follow the
 * reference so that its runtime (src/runtime/moe.c, src/runtime/logits.c) could call this library
 * for that path; every entry cites the reference interface it replaces.
 *
 * Conventions (reference: include/yvex/core.h:13-48, include/yvex/backend.h:1-3):
 *   - every fallible call returns a yvex_status (0 ok, negative error) and fills the caller's
 *     optional yvex_error {code, where, message};
 *   - unsupported work is refused with YVEX_ERR_UNSUPPORTED before any launch; there is no
 *     fallback across backend kinds and no CPU path in this library;
 *   - outputs are published only on success (tensor->is_written, result structs zeroed on failure);
 *   - a backend object and its stream belong to one caller at a time (src/server/scheduler.c:1-8).
 *
 * Struct layouts carry the fields this path reads, under the reference's field names; they are
 * not binary-identical to the reference's structs (those embed planner / identity state that
 * never reaches the backend); a caller inside the reference copies them field by field.
 */
#ifndef YVEX_B200_BACKEND_H
#define YVEX_B200_BACKEND_H
#include <stddef.h>
#include <stdint.h>

#include "yvex_b200_kernels.h"
#ifdef __cplusplus
extern "C" {
#endif

/* ---- status and errors: include/yvex/core.h:13-48 ---------------------------------------- */
typedef enum {
    YVEX_OK = 0, YVEX_ERR = -1, YVEX_ERR_NOMEM = -2, YVEX_ERR_IO = -3, YVEX_ERR_FORMAT = -4,
    YVEX_ERR_UNSUPPORTED = -5, YVEX_ERR_BACKEND = -6, YVEX_ERR_BOUNDS = -7, YVEX_ERR_STATE = -8,
    YVEX_ERR_CANCELLED = -9, YVEX_ERR_INVALID_ARG = -10, YVEX_ERR_TIMEOUT = -11
} yvex_status;
typedef struct { yvex_status code; char where[96]; char message[256]; } yvex_error;
void yvex_error_clear(yvex_error *err);
void yvex_error_set(yvex_error *err, yvex_status code, const char *where, const char *message);
const char *yvex_status_name(yvex_status status);

/* ---- backend object: include/yvex/backend.h:16-152 ---------------------------------------- */
typedef struct yvex_backend yvex_backend;
typedef enum { YVEX_BACKEND_KIND_CPU = 0, YVEX_BACKEND_KIND_CUDA, YVEX_BACKEND_KIND_METAL, YVEX_BACKEND_KIND_ROCM } yvex_backend_kind;
typedef enum { YVEX_BACKEND_STATUS_READY = 0, YVEX_BACKEND_STATUS_CONTEXT_READY, YVEX_BACKEND_STATUS_UNSUPPORTED,
               YVEX_BACKEND_STATUS_FAILED } yvex_backend_status;
typedef struct { yvex_backend_kind kind; const char *device; unsigned long long memory_limit_bytes; } yvex_backend_options;
typedef struct {
    unsigned long long allocated_bytes, allocation_count, allocation_events, release_events;
    unsigned long long h2d_bytes, d2h_bytes, peak_allocated_bytes, memory_limit_bytes;
} yvex_backend_memory_stats;
/* Only YVEX_BACKEND_KIND_CUDA opens (device = "cuda:N" or NULL); every other kind is refused with
 * YVEX_ERR_UNSUPPORTED like the reference does for METAL/ROCM (src/backend/core.c:176-205). */
int yvex_backend_open(yvex_backend **out, const yvex_backend_options *options, yvex_error *err);
int yvex_backend_close_checked(yvex_backend **backend, yvex_error *err);
void yvex_backend_close(yvex_backend *backend);
yvex_backend_kind yvex_backend_kind_of(const yvex_backend *backend);
yvex_backend_status yvex_backend_status_of(const yvex_backend *backend);
int yvex_backend_get_memory_stats(const yvex_backend *backend, yvex_backend_memory_stats *out, yvex_error *err);
int yvex_backend_sync(yvex_backend *backend, yvex_error *err);
/* The CUDA stream the backend enqueues on (for callers that interleave their own work). */
void *yvex_backend_stream(const yvex_backend *backend);

/* ---- tensors: include/yvex/backend.h:44-52,169-192, include/yvex/internal/backend.h:256-269 -- */
typedef enum { YVEX_DTYPE_UNKNOWN = 0, YVEX_DTYPE_F32, YVEX_DTYPE_F16, YVEX_DTYPE_BF16, YVEX_DTYPE_I32, YVEX_DTYPE_U8 } yvex_dtype;
#define YVEX_TENSOR_MAX_DIMS 4
typedef struct {
    const char *name;
    yvex_dtype dtype;
    unsigned int rank;
    unsigned long long dims[YVEX_TENSOR_MAX_DIMS];
    unsigned long long bytes;
} yvex_backend_tensor_desc;
typedef struct yvex_device_tensor {
    yvex_backend *owner;
    unsigned long long owner_id;
    yvex_dtype dtype;
    unsigned int rank;
    unsigned long long dims[YVEX_TENSOR_MAX_DIMS];
    unsigned long long bytes;
    unsigned char *data;          /* device address */
    unsigned char *host_data;     /* pinned staging copy for resident tensors, else NULL */
    int is_written;
} yvex_device_tensor;
int yvex_backend_tensor_alloc(yvex_backend *backend, const yvex_backend_tensor_desc *desc, yvex_device_tensor **out, yvex_error *err);
void yvex_backend_tensor_free(yvex_backend *backend, yvex_device_tensor *tensor);
int yvex_backend_tensor_write(yvex_backend *backend, yvex_device_tensor *tensor, const void *src, unsigned long long len, yvex_error *err);
int yvex_backend_tensor_read(yvex_backend *backend, const yvex_device_tensor *tensor, void *dst, unsigned long long len, yvex_error *err);
unsigned long long yvex_device_tensor_bytes(const yvex_device_tensor *tensor);
int yvex_device_tensor_is_written(const yvex_device_tensor *tensor);

/* ---- resident weights and workspace: include/yvex/internal/backend.h:311-324, src/backend/residency.c:24-112,
 *      src/backend/private.h:159-162 ----------------------------------------------------------------------- */
typedef enum { YVEX_BACKEND_RESIDENT_INVALID = -1, YVEX_BACKEND_RESIDENT_MISS = 0, YVEX_BACKEND_RESIDENT_HIT = 1 } yvex_backend_resident_result;
/* On a discrete GPU the arena is a pinned host staging buffer (host) plus an HBM tensor (out);
 * callers keep naming weights by HOST pointers into the arena, as the reference runtime does. */
int yvex_backend_resident_alloc(yvex_backend *backend, const yvex_backend_tensor_desc *desc, yvex_device_tensor **out,
                                unsigned char **host, yvex_error *err);
/* One H2D copy of the whole arena; synchronous (reference: resident_prefetch). */
int yvex_backend_resident_prefetch(yvex_backend *backend, yvex_device_tensor *tensor, unsigned long long *prefetched_bytes, yvex_error *err);
int yvex_backend_resident_attach(yvex_backend *backend, const unsigned char *host_base, unsigned long long bytes,
                                 const yvex_device_tensor *device_tensor, unsigned long long generation, yvex_error *err);
int yvex_backend_resident_detach(yvex_backend *backend, yvex_error *err);
int yvex_backend_resident_resolve(const yvex_backend *backend, const unsigned char *host, unsigned long long bytes,
                                  unsigned long long *device_address);
int yvex_backend_workspace_attach(yvex_backend *backend, yvex_device_tensor *workspace, yvex_error *err);
int yvex_backend_workspace_detach(yvex_backend *backend, yvex_error *err);

/* Runs the device self-test of the bounded waits (a wait nothing satisfies, `limit_ns` long) and
 * reports it the way every expired device wait is reported: YVEX_ERR_TIMEOUT, backend still READY.
 * Any other outcome is YVEX_ERR_BACKEND. No reference counterpart. */
int yvex_backend_selftest_bounded_wait(yvex_backend *backend, unsigned long long limit_ns, unsigned long long *elapsed_ns,
                                       yvex_error *err);

/* ---- capability: include/yvex/backend.h:77-129 ------------------------------------------------------------ */
typedef enum {
    YVEX_BACKEND_VARIANT_ATTENTION_CAUSAL_F32 = 13, YVEX_BACKEND_VARIANT_ATTENTION_NONCAUSAL_F32 = 14,
    YVEX_BACKEND_VARIANT_QTYPE_ROW_DOT = 15, YVEX_BACKEND_VARIANT_ATTENTION_ENCODED = 16, YVEX_BACKEND_VARIANT_COUNT = 17
} yvex_backend_operation_variant;
typedef enum { YVEX_BACKEND_CAPABILITY_UNSUPPORTED = 0, YVEX_BACKEND_CAPABILITY_SUPPORTED, YVEX_BACKEND_CAPABILITY_FAILED } yvex_backend_capability_state;
typedef struct { yvex_backend_kind backend_kind; int variant; yvex_backend_capability_state state; int context_available, function_available; } yvex_backend_capability_result;
int yvex_backend_query_capability(const yvex_backend *backend, int variant, yvex_backend_capability_result *out, yvex_error *err);
/* 1 if qtype has decode + device compute here (the reference's dedicated_cuda_compute_available,
 * src/gguf/quant_registry.c:50-103, plus the declared Q4_K extension). */
int yvex_backend_qtype_supported(const yvex_backend *backend, unsigned int qtype);

/* ---- vtable ops that are NOT on this path fail closed: src/backend/core.c:954-958 -------------------------- */
int yvex_backend_op_embed(yvex_backend *backend, const yvex_device_tensor *embedding, const unsigned int *token_ids,
                          unsigned long long token_count, yvex_device_tensor *out, yvex_error *err);
int yvex_backend_op_rms_norm(yvex_backend *backend, const yvex_device_tensor *input, const yvex_device_tensor *weight, float epsilon,
                             yvex_device_tensor *out, yvex_error *err);
int yvex_backend_op_matmul(yvex_backend *backend, const yvex_device_tensor *input, const yvex_device_tensor *weight,
                           yvex_device_tensor *out, yvex_error *err);

/* ---- encoded matvec: include/yvex/internal/backend.h:325-337, src/backend/cuda/qtype.c:220-405 ------------- */
typedef struct yvex_backend_cuda_operation_facts {
    unsigned long long h2d_bytes, d2h_bytes, d2d_bytes, kernel_launches, upload_count;
    unsigned long long download_count, stream_synchronizations, device_synchronizations;
    unsigned long long active_weight_bytes, state_bytes;
    unsigned long long activation_bytes, temporary_bytes, tensor_core_launches;
    int compulsory_memory_facts_available;
} yvex_backend_cuda_operation_facts;
/* output[input_row][row] = dot(row, input[input_row]) (+ additive). resident_encoded is a HOST pointer
 * into the attached resident arena. Synchronises like the reference. The reference's two variants:
 *   activation_q8 = 1  for IQ2_XXS, Q2_K, Q8_0 and MXFP4 rows of a width that is a multiple of 256 the input
 *                      rows go through the Q8_K quantiser first (src/backend/cuda/qtype.c:252-253; other
 *                      qtypes, widths or a split input take the plain path, as there): the result is the
 *                      product with the de-quantised activations, within 1e-5 (1 + |.|) of the CPU codec
 *                      on those values like the reference's own (tests/unit/cuda/quant_qtype.c:389-396);
 *   input_tail         the row is input[0 : input_head_width] ++ input_tail, rounded to bf16
 *                      (yvex_qtype_split_matvec, src/backend/cuda/kernels.cu:736-781). */
int yvex_backend_cuda_encoded_matvec(yvex_backend *backend, const unsigned char *resident_encoded,
    unsigned long long encoded_bytes, unsigned int qtype, unsigned long long row_count,
    unsigned long long row_width, unsigned long long row_bytes, unsigned long long input_rows,
    const yvex_device_tensor *input, const yvex_device_tensor *input_tail, unsigned long long input_head_width,
    const yvex_device_tensor *additive, yvex_device_tensor *output, int activation_q8,
    yvex_backend_cuda_operation_facts *facts, yvex_error *err);

/* Decodes selected rows of a resident matrix into a backend-owned F32 tensor [selected_rows x row_width]
 * (src/backend/cuda/qtype.c:404-520): row_ids is a HOST array, an id >= row_count is YVEX_ERR_BOUNDS. */
int yvex_backend_cuda_encoded_gather(yvex_backend *backend, const unsigned char *resident_encoded,
    unsigned long long encoded_bytes, unsigned int qtype, unsigned long long row_count, unsigned long long row_width,
    unsigned long long row_bytes, const unsigned int *row_ids, unsigned long long selected_rows, yvex_device_tensor *output,
    yvex_backend_cuda_operation_facts *facts, yvex_error *err);

/* ---- attention: include/yvex/backend.h:246-257 (public op) ------------------------------------------------- */
/*
 * One encoded row times one f32 vector, both HOST memory, result to host: yvex_cuda_quant_row_dot
 * (src/backend/cuda/private.h:588-596, src/backend/cuda/qtype.c:527-700). `failure` (optional) is zeroed on
 * success and filled on every refusal as the reference fills it (code, expected, actual, qtype; the index
 * fields all-ones, operation = the operation count): INVALID_ARGUMENT for missing or misaligned pointers,
 * CUDA_COMPUTE_UNAVAILABLE + YVEX_ERR_UNSUPPORTED for a qtype without a device decoder (here Q4_K has one),
 * ROW_DIVISIBILITY / BYTE_OVERFLOW + YVEX_ERR_BOUNDS for a row that is not whole blocks or whose byte count
 * differs, WORKER for a failed copy or launch, NONFINITE + YVEX_ERR_FORMAT for a malformed block scale.
 * The YVEX_TEST_CUDA_QTYPE_COPY_FAILURE=input|output seams fail the call before / after the device work.
 */
typedef enum {
    YVEX_QUANT_FAILURE_NONE = 0, YVEX_QUANT_FAILURE_INVALID_ARGUMENT = 1, YVEX_QUANT_FAILURE_CUDA_COMPUTE_UNAVAILABLE = 21,
    YVEX_QUANT_FAILURE_ROW_DIVISIBILITY = 28, YVEX_QUANT_FAILURE_BYTE_OVERFLOW = 30, YVEX_QUANT_FAILURE_NONFINITE = 37,
    YVEX_QUANT_FAILURE_WORKER = 45, YVEX_QUANT_FAILURE_CLEANUP = 46
} yvex_quant_failure_code;                       /* the values of include/yvex/internal/quant_numeric.h:31-82 that this backend reports */
#define YVEX_TRANSFORM_OP_COUNT 9                /* include/yvex/internal/compilation.h:112-122 */
typedef struct yvex_quant_failure {
    int code;                                    /* yvex_quant_failure_code */
    unsigned long long terminal_ordinal, source_index, row_index, block_index, expected, actual;
    unsigned int qtype;
    int operation;                               /* yvex_transform_operation_kind */
} yvex_quant_failure;
int yvex_cuda_quant_row_dot(yvex_backend *backend, unsigned int qtype, const unsigned char *encoded, size_t encoded_bytes,
                            const float *vector, unsigned long long elements, float *out, yvex_quant_failure *failure, yvex_error *err);
int yvex_backend_op_attention(yvex_backend *backend, const yvex_device_tensor *query, const yvex_device_tensor *keys,
                              const yvex_device_tensor *values, unsigned long long seq_len, unsigned long long position,
                              float scale, int causal, yvex_device_tensor *score_scratch,
                              yvex_device_tensor *probability_scratch, yvex_device_tensor *out, yvex_error *err);
/* Extension (the reference's GQA exists only as the text-encoder prefill kernel,
 * src/backend/cuda/transformer_kernels.cu:85-145): decode-time GQA over a bf16 KV cache.
 * query [sessions][q_heads][head_dim] bf16, keys/values [sessions][kv_heads][context][head_dim] bf16,
 * out [sessions][q_heads][head_dim] f32. Scratch comes from the attached workspace. */
int yvex_backend_attention_gqa_decode(yvex_backend *backend, const yvex_device_tensor *query, const yvex_device_tensor *keys,
                                      const yvex_device_tensor *values, unsigned long long sessions, unsigned long long q_heads,
                                      unsigned long long kv_heads, unsigned long long head_dim, unsigned long long context,
                                      unsigned long long position, float scale, yvex_device_tensor *out, yvex_error *err);

/* ---- MoE op table: include/yvex/internal/moe.h:36-84,161-166,221-297 --------------------------------------- */
#define YVEX_MOE_MAX_SELECTED 16u
#define YVEX_MOE_KERNEL_SM100_DEQUANT_GEMV "sm100-dequant-gemv"
#define YVEX_MOE_KERNEL_SM100_TCGEN05_EXPERT "sm100-f16-tcgen05-expert"
typedef enum { YVEX_MOE_ROUTER_HASH_TOKEN_ID = 0, YVEX_MOE_ROUTER_LEARNED_HIDDEN_STATE } yvex_moe_router_class;
typedef enum {
    YVEX_MOE_WEIGHT_FFN_NORM = 0, YVEX_MOE_WEIGHT_MHC_FUNCTION, YVEX_MOE_WEIGHT_MHC_BASE, YVEX_MOE_WEIGHT_MHC_SCALE,
    YVEX_MOE_WEIGHT_ROUTER, YVEX_MOE_WEIGHT_ROUTER_TABLE, YVEX_MOE_WEIGHT_ROUTER_BIAS, YVEX_MOE_WEIGHT_ROUTED_GATE,
    YVEX_MOE_WEIGHT_ROUTED_UP, YVEX_MOE_WEIGHT_ROUTED_DOWN, YVEX_MOE_WEIGHT_SHARED_GATE, YVEX_MOE_WEIGHT_SHARED_UP,
    YVEX_MOE_WEIGHT_SHARED_DOWN, YVEX_MOE_WEIGHT_COUNT
} yvex_moe_weight_slot;
/*
 * The structs below are laid out field for field as the reference's (include/yvex/internal/moe.h:54-84,
 * :182-271, include/yvex/internal/execution.h:329-333, include/yvex/internal/execution_batch.h:126-137),
 * so a caller compiled against the reference's headers can pass its own objects: no field-copying
 * adaptor. Enumerations this backend does not interpret are declared as `int` (the same size and
 * alignment); fields it does not use are ignored, not removed. tests/abi_probe.c prints every size and
 * offset and is compared with the table the same file produced against the reference's headers.
 */
#define YVEX_RUNTIME_DESCRIPTOR_QTYPE_CAP 43u
#define YVEX_SHA256_HEX_CAP 65u                  /* include/yvex/artifact.h:68 */
#define YVEX_MOE_ROW_BATCH_SCHEMA_V1 1u
#define YVEX_MOE_ROW_BATCH_RESULT_SCHEMA_V4 4u
/* Extension: a row batch whose schema_version is this value is a yvex_moe_row_batch_logits. */
#define YVEX_MOE_ROW_BATCH_SCHEMA_B200_LOGITS 0x42320001u
typedef enum { YVEX_EXECUTION_CLASS_PORTABLE_REFERENCE = 0, YVEX_EXECUTION_CLASS_DEVICE_NATIVE, YVEX_EXECUTION_CLASS_FORENSIC_REFERENCE } yvex_execution_class;
typedef enum { YVEX_EXECUTION_LAYOUT_CANONICAL_ROW = 0, YVEX_EXECUTION_LAYOUT_CONTIGUOUS_DENSE, YVEX_EXECUTION_LAYOUT_EXPERT_MAJOR,
               YVEX_EXECUTION_LAYOUT_DERIVED_BACKEND } yvex_execution_layout_class;
typedef struct yvex_execution_batch yvex_execution_batch;                 /* only ever pointed to */
typedef struct yvex_execution_batch_source yvex_execution_batch_source;
typedef struct yvex_execution_batch_row yvex_execution_batch_row;
typedef struct yvex_expert_worklist_policy yvex_expert_worklist_policy;
typedef struct {
    unsigned long long active_weight_bytes, state_bytes, activation_bytes, temporary_bytes;
    unsigned long long measured_operations, missing_operations;
    int complete;
} yvex_execution_memory_facts;
typedef struct {
    unsigned long long tensor_id, expert_index;
    int role;                            /* yvex_tensor_role */
    unsigned int qtype;
    yvex_execution_layout_class layout;  /* a backend-derived layout is refused: none is offered */
    int activation;                      /* yvex_execution_activation_class */
    const char *kernel_family;           /* NULL or one of the YVEX_MOE_KERNEL_SM100_* names; others are refused */
    const unsigned char *encoded;        /* HOST pointer into the resident arena */
    size_t encoded_bytes, storage_bytes;
    unsigned long long row_bytes, row_width, row_count;
    unsigned long long device_address;   /* when non-zero, used as is (src/backend/cuda/moe.c:235-236); else `encoded` is resolved */
} yvex_moe_weight_view;
typedef struct {
    unsigned int schema_version;
    unsigned long long ordinal, layer_index, predictor_index;
    int tensor_scope;                    /* yvex_tensor_scope */
    yvex_moe_router_class router_class;
    int scoring, topk_policy, activation;     /* sqrt-softplus / no-aux top-k / SiLU: the only values (include/yvex/internal/moe.h:35-37) */
    /* residual_streams > 1 selects the mHC envelope: rows are expanded_width = residual_streams *
     * hidden_width wide on both sides, the FFN_NORM / MHC_FUNCTION / MHC_BASE / MHC_SCALE weight slots
     * are required and mhc_mixing_rows = (residual_streams + 2) * residual_streams. */
    unsigned long long hidden_width, residual_streams, expanded_width;
    unsigned long long mhc_mixing_rows, mhc_sinkhorn_iterations;
    unsigned long long routed_experts, shared_experts, experts_per_token;
    unsigned long long expert_intermediate_width, shared_intermediate_width;
    unsigned long long hash_table_rows, hash_table_columns, correction_bias_width;
    double rms_epsilon, mhc_epsilon, mhc_post_multiplier;
    double routed_scaling_factor, activation_limit;
    int requires_token_ids, requires_correction_bias, normalize_topk_probabilities;
    unsigned long long tensor_ids[YVEX_MOE_WEIGHT_COUNT];
    unsigned int qtypes[YVEX_MOE_WEIGHT_COUNT];
    char layer_identity[YVEX_SHA256_HEX_CAP];
} yvex_moe_layer_plan;
/* Pointer-free worklist summary, laid out as include/yvex/internal/execution_batch.h:126-137. */
typedef yvex_b200_worklist_observation yvex_expert_worklist_observation;
typedef struct {
    unsigned long long row_count, row_expert_pairs;
    yvex_expert_worklist_observation worklist;       /* with the status word in deferred mode (src/backend/cuda/moe.c:1710-1716): filled by complete_rows */
    unsigned long long tensor_core_executed_pairs;
    unsigned long long routed_experts, active_base_bytes, active_per_expert_bytes;
    unsigned long long activation_bytes, temporary_bytes;
    int status, pending;
} yvex_moe_device_completion_slot;
typedef struct { int defer; yvex_moe_device_completion_slot *host; } yvex_moe_device_completion;
typedef struct {
    const yvex_moe_layer_plan *layer;
    yvex_moe_weight_view weights[YVEX_MOE_WEIGHT_COUNT];
    const float *expanded_input;               /* single-token entry points only; unused by the row-batch table */
    const yvex_device_tensor *device_input;
    yvex_device_tensor *device_output;
    unsigned int token_id;
    int token_id_present;
    int (*cancel_requested)(void *context);
    void *cancel_context;
    int evidence_level;                        /* yvex_attention_evidence_level; FULL (3) is refused like the reference's width-N path */
    int eager_execution;
    const yvex_moe_device_completion *device_completion;
    const yvex_execution_batch *execution_batch;
    const yvex_expert_worklist_policy *worklist_policy;
} yvex_moe_layer_job;
typedef struct {
    unsigned int schema_version;               /* YVEX_MOE_ROW_BATCH_SCHEMA_V1, or the logits extension below */
    unsigned long long row_count, row_width, row_stride;
    const float *expanded_rows;                /* host rows (copied in), or NULL when device_rows is given */
    const yvex_device_tensor *device_rows;     /* f32 [row_count x row_stride] */
    yvex_device_tensor *device_outputs;        /* f32 [row_count x row_stride], optional when host output is given */
    const unsigned int *token_ids;
    int token_ids_present;
    int provenance;                            /* yvex_execution_batch_provenance: counted in the worklist summary */
    unsigned int phase;
    yvex_execution_class execution_class;
    const char *execution_profile_identity;
    const yvex_execution_batch_source *execution_sources;
    const yvex_execution_batch_row *execution_rows;
    unsigned long long execution_source_count;
    int complete_after_operation;
} yvex_moe_row_batch;
/* Extension: router logits supplied by the caller replace the router projection. base.schema_version
 * must be YVEX_MOE_ROW_BATCH_SCHEMA_B200_LOGITS; the table's entry points take a pointer to `base`. */
typedef struct {
    yvex_moe_row_batch base;
    const float *router_logits;                /* host [row_count x routed_experts] */
    const yvex_device_tensor *device_router_logits;
} yvex_moe_row_batch_logits;
typedef struct {
    /* host arrays, each optional here (the reference's width-N path requires all of them): the combined rows,
     * the f32 rank-ordered routed sum and the shared expert's row [row_count x hidden_width], and with the
     * mHC envelope its post gates [row_count x streams] and combination matrices [row_count x streams^2] */
    float *combined_rows, *routed_rows, *shared_rows, *post_rows, *combination_rows;
    unsigned long long combined_capacity, routed_capacity, shared_capacity;
    unsigned long long post_capacity, combination_capacity;
    unsigned long long *selected_experts;      /* host [row_count x experts_per_token], optional */
    float *selected_weights;
    unsigned long long selection_capacity;
} yvex_moe_row_batch_output;
typedef struct {
    unsigned int schema_version;
    int completed, execution_profile_available, device_completion_pending;
    yvex_execution_class execution_class;
    unsigned long long row_count, row_expert_pairs, unique_experts;
    yvex_expert_worklist_observation worklists;
    unsigned long long grouped_expert_operations, shared_expert_operations;
    unsigned long long expert_subviews_accessed, encoded_bytes_read;
    unsigned long long h2d_bytes, d2h_bytes, d2d_bytes, kernel_launches;
    unsigned long long tensor_core_launches;
    unsigned long long graph_launches, graph_captures, graph_replays;
    unsigned long long upload_count, download_count, cache_hits, cache_misses;
    unsigned long long stream_synchronizations, device_synchronizations;
    unsigned long long active_weight_base_bytes;
    unsigned long long active_weight_per_unique_expert_bytes;
    yvex_execution_memory_facts memory;        /* active weight bytes (each byte once), activation and temporary bytes */
    unsigned long long total_ns, synchronization_ns;
    char execution_profile_identity[YVEX_SHA256_HEX_CAP];
    char execution_batch_identity[YVEX_SHA256_HEX_CAP];
    char worklist_policy_identity[YVEX_SHA256_HEX_CAP];
    char expert_worklist_identity[YVEX_SHA256_HEX_CAP];
    char routing_digest[YVEX_SHA256_HEX_CAP];
    char execution_identity[YVEX_SHA256_HEX_CAP];
} yvex_moe_row_batch_result;
typedef struct {
    /* Derived layouts are not offered: both return YVEX_ERR_UNSUPPORTED and the canonical row layout is used. */
    int (*derived_layout_plan)(const void *decision, unsigned long long *storage_bytes, yvex_error *err);
    int (*derived_layout_build)(const void *decision, const unsigned char *canonical, unsigned long long canonical_bytes,
                                unsigned char *derived, unsigned long long storage_bytes, yvex_error *err);
    int (*workspace_required)(const yvex_moe_layer_plan *layer, unsigned long long row_count, unsigned long long *bytes, yvex_error *err);
    /* <= 62 rows, like moe_cuda_execute_rows (src/backend/cuda/moe.c:1826-1923). */
    int (*execute_rows)(yvex_backend *backend, const yvex_moe_layer_job *job, const yvex_moe_row_batch *batch,
                        const yvex_moe_row_batch_output *output, yvex_moe_row_batch_result *result, yvex_error *err);
    int (*complete_rows)(yvex_backend *backend, int barrier_observed, yvex_moe_row_batch_result *result, yvex_error *err);
    /* Extension: the same contract without the row limit (prefill); workspace_required_wide sizes it. */
    int (*workspace_required_wide)(const yvex_moe_layer_plan *layer, unsigned long long row_count, unsigned long long *bytes, yvex_error *err);
    int (*execute_rows_wide)(yvex_backend *backend, const yvex_moe_layer_job *job, const yvex_moe_row_batch *batch,
                             const yvex_moe_row_batch_output *output, yvex_moe_row_batch_result *result, yvex_error *err);
} yvex_backend_moe_operations;
/*
 * Token-local MoE transaction (include/yvex/internal/moe.h:160-166, :198-214, :308-319;
 * src/backend/cuda/moe.c:504-848; caller src/runtime/moe.c:647-694): one token, one expert per call.
 *   begin       uploads job->expanded_input (or reads job->device_input), runs the envelope's prepare step
 *               (or, without an envelope, the bf16 ingress rounding), the router projection, scoring and top-k,
 *               and publishes result->router. When the caller will not add the routed experts itself (a
 *               device output, evidence below FULL and device addresses on all three routed packs: the
 *               condition at src/runtime/moe.c:654-658) begin adds the selected experts.
 *   add_expert  gate and up matvecs of the normalized row, SwiGLU * weight -> bf16, down matvec -> bf16, added to
 *               the routed (f32, call order) or shared aggregate. Weights must be resident on the backend
 *               (YVEX_ERR_STATE otherwise); any qtype with a device decoder is taken.
 *   finish      combined = bf16(routed + shared), the envelope's post step into job->device_output when there is
 *               one, downloads (everything without a device output or at FULL evidence; the selection
 *               otherwise), one synchronisation, the status word, the counters.
 *   close       frees the transaction; nothing of the backend is released.
 * Scratch comes from the attached workspace (workspace_required(layer, 1) covers it) and is reset by begin,
 * like backend_workspace_reset in the reference: one transaction at a time per backend.
 */
typedef struct {
    unsigned long long selected_count;
    unsigned long long selected_experts[YVEX_MOE_MAX_SELECTED];
    float router_logits[256], router_scores[256];
    float selected_weights[YVEX_MOE_MAX_SELECTED];
} yvex_moe_router_result;
typedef struct {
    float *combined_output, *post, *combination;
    unsigned long long combined_capacity, post_capacity, combination_capacity;
    float *routed_output, *shared_output;
    unsigned long long routed_capacity, shared_capacity;
    yvex_moe_router_result router;
    unsigned long long expert_subviews_accessed, encoded_bytes_read;
    unsigned long long host_to_device_bytes, device_to_host_bytes, kernel_launches;
    unsigned long long cache_hits, cache_misses, upload_count, download_count;
    unsigned long long stream_synchronizations, device_synchronizations, device_to_device_bytes;
    yvex_execution_memory_facts memory;
    unsigned long long ingress_ns, routing_ns, routed_ns, shared_ns, post_ns, total_ns;
    unsigned long long synchronization_ns;
    unsigned long long qtype_counts[YVEX_RUNTIME_DESCRIPTOR_QTYPE_CAP];
    char routed_digest[YVEX_SHA256_HEX_CAP], shared_digest[YVEX_SHA256_HEX_CAP];
    char combined_digest[YVEX_SHA256_HEX_CAP], routing_digest[YVEX_SHA256_HEX_CAP];
} yvex_moe_layer_result;
typedef struct yvex_backend_moe_execution yvex_backend_moe_execution;
int yvex_backend_moe_begin(yvex_backend_moe_execution **out, yvex_backend *backend, const yvex_moe_layer_job *job,
                           yvex_moe_layer_result *result, yvex_error *err);
int yvex_backend_moe_add_expert(yvex_backend_moe_execution *execution, const yvex_moe_weight_view *gate,
                                const yvex_moe_weight_view *up, const yvex_moe_weight_view *down, float route_weight,
                                int shared, yvex_error *err);
int yvex_backend_moe_finish(yvex_backend_moe_execution *execution, yvex_moe_layer_result *result, yvex_error *err);
int yvex_backend_moe_close(yvex_backend_moe_execution **execution, yvex_error *err);
/*
 * Expert-parallel layer over the ranks of one box, one process per GPU (no reference counterpart: the reference is
 * single-device). Rank r owns the tokens it passes in and the routed experts [r * E / world, (r + 1) * E / world):
 * the job's layer plan describes the WHOLE layer (routed_experts = E), its routed weight views hold the rank's
 * shard (E / world experts), the shared expert's and the router's views are the same on every rank. One call runs
 * one layer for the rank's rows: router and top-k here, pairs dispatched to their experts' ranks and results brought
 * back by all-to-all-v exchanges made of ncclSend / ncclRecv groups, rank-ordered combination here. Every rank must
 * make the call; rows may differ between ranks.
 *   yvex_moe_ep_unique_id   rank 0 creates the communicator's identifier (ncclGetUniqueId) and hands it to the
 *                           other ranks by any means of the application (a file, a socket)
 *   yvex_moe_ep_open        joins the communicator (blocks until every rank has joined); deadline_ms bounds every
 *                           later wait for a peer
 *   yvex_moe_ep_workspace_required / yvex_backend_workspace_attach size and provide the device scratch
 *   yvex_moe_ep_execute_rows host rows in (batch->expanded_rows, hidden wide; router logits through the
 *                           yvex_moe_row_batch_logits extension, or resident F32 router weights), host rows out
 *                           (output->combined_rows; the selection when asked for). A peer that does not take part
 *                           before the deadline aborts the communicator: YVEX_ERR_TIMEOUT now, YVEX_ERR_STATE on
 *                           every later call; the backend itself stays usable.
 * NCCL is loaded at run time (libnccl.so.2, or the path in YVEX_B200_NCCL_LIBRARY): YVEX_ERR_UNSUPPORTED without it.
 */
#define YVEX_MOE_EP_ID_BYTES 128
typedef struct yvex_moe_ep yvex_moe_ep;
int yvex_moe_ep_unique_id(unsigned char id[YVEX_MOE_EP_ID_BYTES], yvex_error *err);
int yvex_moe_ep_open(yvex_moe_ep **out, yvex_backend *backend, const unsigned char id[YVEX_MOE_EP_ID_BYTES], unsigned int world,
                     unsigned int rank, unsigned long long deadline_ms, yvex_error *err);
int yvex_moe_ep_workspace_required(const yvex_moe_layer_plan *layer, unsigned long long rows, unsigned int world, unsigned long long *bytes,
                                   yvex_error *err);
int yvex_moe_ep_execute_rows(yvex_moe_ep *ep, const yvex_moe_layer_job *job, const yvex_moe_row_batch *batch,
                             const yvex_moe_row_batch_output *output, yvex_moe_row_batch_result *result, yvex_error *err);
int yvex_moe_ep_close(yvex_moe_ep **ep, yvex_error *err);
/* "sizeof type N" / "offsetof type.field N" lines for every entry of yvex_b200_abi_fields.h, as this
 * library was compiled; a binding compares its own table with it. No reference counterpart. */
const char *yvex_backend_abi_layout(void);
/* Row ranges whose host copies overlapped compute in the last execute_rows_wide call (0: the call did
 * not use the copy pipeline). No reference counterpart. */
unsigned long long yvex_backend_moe_last_pipeline_chunks(const yvex_backend *backend);
/* NULL unless the backend is an open CUDA backend (src/backend/cuda/moe.c:1968-1981). */
const yvex_backend_moe_operations *yvex_backend_moe_operations_get(const yvex_backend *backend);

/* ---- external MoE input fixtures: include/yvex/internal/moe.h:120-160, src/runtime/moe_input.c ------------- */
#define YVEX_MOE_INPUT_SUFFIX ".yvex-moe-input"
typedef struct {
    unsigned int schema_version;
    unsigned long long token_start, token_count, layer_count;
    unsigned long long activation_payload_bytes, token_id_payload_bytes;
    char logical_model_identity[YVEX_SHA256_HEX_CAP];
    char runtime_numeric_identity[YVEX_SHA256_HEX_CAP];
    char runtime_descriptor_identity[YVEX_SHA256_HEX_CAP];
    char moe_plan_identity[YVEX_SHA256_HEX_CAP];
    char activation_payload_digest[YVEX_SHA256_HEX_CAP];
    char token_id_payload_digest[YVEX_SHA256_HEX_CAP];
    char input_identity[YVEX_SHA256_HEX_CAP];
} yvex_moe_input_summary;
typedef struct {
    unsigned long long ordinal, layer_index, width, stride;
    unsigned long long payload_offset, payload_bytes;
    char layer_identity[YVEX_SHA256_HEX_CAP];
} yvex_moe_input_layer_record;
typedef struct yvex_moe_input yvex_moe_input;
typedef struct { unsigned long long maximum_file_bytes; } yvex_moe_input_limits;
/* Opens and verifies a fixture file (regular, not a symbolic link, at most limits->maximum_file_bytes):
 * sizes, ordering, finite activations, both payload digests and the input identity (src/runtime/moe_input.c:279-412). */
int yvex_moe_input_open_file(yvex_moe_input **out, const char *path, const yvex_moe_input_limits *limits, yvex_error *err);
/* The same admission for a serialized fixture already in memory (copied; the caller keeps its buffer). */
int yvex_moe_input_open_image(yvex_moe_input **out, const void *image, unsigned long long bytes, yvex_error *err);
const yvex_moe_input_summary *yvex_moe_input_summary_get(const yvex_moe_input *input);
const yvex_moe_input_layer_record *yvex_moe_input_layer_record_at(const yvex_moe_input *input, unsigned long long ordinal);
int yvex_moe_input_layer_view(const yvex_moe_input *input, unsigned long long ordinal, const float **values,
                              unsigned long long *stride, yvex_error *err);
const unsigned int *yvex_moe_input_token_ids(const yvex_moe_input *input);
void yvex_moe_input_close(yvex_moe_input **input);
/* The rows of one fixture layer as the host-row batch execute_rows / execute_rows_wide take
 * (what the reference's `graph execute moe` operator feeds the backend, src/runtime/moe.c:1290-1330). */
int yvex_moe_input_row_batch(const yvex_moe_input *input, unsigned long long ordinal, yvex_moe_row_batch *batch, yvex_error *err);

#ifdef __cplusplus
}
#endif
#endif
