/*
 * yvex_b200 device layer: the thin C-ABI shim over the hand-written sm_100a kernels.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (passed as void* so C11
 * callers need no CUDA headers), enqueues its kernels on that stream and returns immediately
 * with a yvex_status value (0 ok, negative = refusal BEFORE any launch). Nothing here allocates,
 * synchronises or copies to the host. Numerical and argument faults found on the device are
 * reported through the caller's `int *status` word with the reference's convention
 * (src/backend/cuda/moe.c:293-295): 0 ok, 1 non-finite numerics, 2 invalid arguments,
 * 3 bounded wait expired; kernels return early once it is non-zero.
 *
 * Unsupported qtypes fail closed at entry with YVEX_ERR_UNSUPPORTED (-5): the admitted set is
 * the reference's registry (src/gguf/quant_registry.c:50-103) - F32, F16, BF16, Q8_0, Q2_K,
 * IQ2_XXS - plus Q4_K, which the reference stores but cannot decode; Q4_K is this library's
 * declared extension and is compiled in only because the benchmark configs name it.
 */
#ifndef YVEX_B200_KERNELS_H
#define YVEX_B200_KERNELS_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

#define YVEX_B200_STATUS_OK 0
#define YVEX_B200_STATUS_NUMERIC 1
#define YVEX_B200_STATUS_ARGUMENT 2
#define YVEX_B200_STATUS_TIMEOUT 3

/* Library identity; also the cheapest way to prove the shared object loaded. */
const char *yvex_b200_version(void);
/* 1 if `qtype` has a device decoder/dot in this library, else 0 (fail-closed answer). */
int yvex_b200_qtype_supported(unsigned int qtype);
/* Block geometry of the reference's table (src/gguf/qtype.c:15-104); 0 on unknown id. */
int yvex_b200_qtype_geometry(unsigned int qtype, unsigned int *block_elements,
                             unsigned int *block_bytes);

/*
 * Accounting the reference keeps in yvex_backend_cuda_operation_facts.kernel_launches
 * (include/yvex/internal/backend.h:325-331): kernels this library has enqueued since load.
 */
unsigned long long yvex_b200_launch_count(void);
/*
 * Optional per-phase timing, the device-side counterpart of the reference's per-phase
 * nanosecond counters (include/yvex/internal/moe.h:209-210). While `events` (an array of
 * `count` cudaEvent_t handles owned by the caller) is registered, the MoE entry points record
 * events[0] when they start and events[i] after phase i (1 route, 2 gate/up, 3 down+combine for
 * the narrow path; 1 route, 2 permute+gather, 3 gate/up GEMM, 4 SwiGLU + down GEMM, 5 combine
 * for the wide path).
 * Pass count 0 to unregister. Process-wide; not meant for concurrent callers.
 */
int yvex_b200_phase_events(void **events, int count);

/*
 * Elementwise decode of encoded rows to f32, bit-exact with yvex_quant_decode_block
 * (src/gguf/quant_block.c:769-881). Replaces yvex_encoded_row_decode
 * (src/backend/cuda/kernels.cu:784-800). out is [rows x width].
 */
int yvex_b200_dequant_rows(unsigned int qtype, const void *encoded, uint64_t rows, uint64_t width,
                           uint64_t row_bytes, float *out, int *status, void *stream);
/* The same for selected rows: out row i = decoded matrix row row_ids[i] (device array, ids < rows or
 * status 2). Replaces yvex_qtype_gather behind yvex_backend_cuda_encoded_gather
 * (src/backend/cuda/qtype.c:404-520). out is [selected_rows x width]. */
int yvex_b200_dequant_gather(unsigned int qtype, const void *encoded, uint64_t rows, uint64_t width, uint64_t row_bytes,
                             const uint32_t *row_ids, uint64_t selected_rows, float *out, int *status, void *stream);
/* Activation rows as the reference's Q8_K activation path sees them: per 256 values the element of
 * largest magnitude sets inverse = -127 / value, each value becomes rint(inverse * x) clamped to
 * [-128, 127], divided by inverse again (quantiser src/backend/cuda/kernels.cu:436-489; the definition
 * of its results tests/unit/cuda/quant_qtype.c:161-186). width % 256 == 0, 16-byte aligned rows. */
int yvex_b200_q8k_round_trip(const float *x, uint64_t rows, uint64_t width, float *out, int *status, void *stream);
/* out[r] = bf16(head[r] ++ tail[r]) with head_width and width - head_width values: the input row of the
 * reference's split-input matvec (src/backend/cuda/kernels.cu:736-781). */
int yvex_b200_concat_bf16(const float *head, const float *tail, uint64_t head_width, uint64_t width, uint64_t rows,
                          float *out, int *status, void *stream);

/*
 * Dequant-fused matvec: out[i][r] = dot(row r, input[i]) (+ additive[i][r]), optional bf16
 * rounding of the result. Replaces yvex_qtype_matvec (src/backend/cuda/kernels.cu:529-626);
 * CPU meaning: a loop of yvex_quant_cpu_dot (src/gguf/quant_compute.c:116-181).
 * input is [input_rows x width] f32, out is [input_rows x rows] f32.
 * Stream order: the block-qtype kernels are launched with programmatic stream serialization and
 * prefetch encoded rows before the kernel launched before them on the stream has finished; input,
 * additive and out are only touched after it has. So the encoded rows must not be the output of
 * the immediately preceding kernel on the same stream (weights resident before the step are fine).
 */
int yvex_b200_gemv(unsigned int qtype, const void *encoded, uint64_t rows, uint64_t width,
                   uint64_t row_bytes, const float *input, uint64_t input_rows,
                   const float *additive, float *out, int round_bf16, int *status, void *stream);

/*
 * A batch of independent matvecs of one shape in one launch: matrix m is the canonical row layout at
 * encoded + m * matrix_stride, its input vector at input + m * input_stride (f32 elements), its
 * result (and optional additive row) at out + m * out_stride. What a decode step does for several
 * projections or experts of one geometry at once; no reference counterpart (the reference issues
 * one yvex_qtype_matvec per matrix, src/backend/cuda/qtype.c:340-379). IQ2_XXS, Q4_K and Q8_0 with
 * width a multiple of 256 (<= 8192), a 16-byte aligned base and stride run on the persistent
 * streaming kernel; everything else falls back to one yvex_b200_gemv per matrix.
 */
int yvex_b200_gemv_batch(unsigned int qtype, const void *encoded, uint64_t matrix_stride, uint64_t count,
                         uint64_t rows, uint64_t width, uint64_t row_bytes, const float *input,
                         uint64_t input_stride, const float *additive, float *out, uint64_t out_stride,
                         int round_bf16, int *status, void *stream);

/* Geometry and policy of one MoE FFN layer: the fields of yvex_moe_layer_plan
 * (include/yvex/internal/moe.h:54-84) that the execution path reads. */
typedef struct {
    uint64_t hidden, experts, topk, inter, shared_inter;
    double scaling, limit;          /* routed_scaling_factor, activation_limit */
    int normalize;                  /* normalize_topk_probabilities */
    int router_class;               /* 1 learned hidden-state, 0 token-id hash table */
    unsigned int gate_qtype, up_qtype, down_qtype;
    uint64_t hash_rows, hash_stored_rows;
} yvex_b200_moe_geometry;

/* Device addresses of the layer's weights (canonical row layout, routed packs expert-major:
 * expert e at byte offset e * rows_per_expert * row_bytes, src/backend/cuda/moe.c:617-619). */
typedef struct {
    const float *router;            /* [experts x hidden] f32, NULL when logits are supplied */
    const float *bias;              /* [experts] f32 or NULL */
    const int32_t *hash_table;      /* [hash_stored_rows x topk] or NULL */
    const void *gate, *up, *down;
    const void *shared_gate, *shared_up, *shared_down;
} yvex_b200_moe_weights;

/* Bytes of 256-byte-aligned device scratch the MoE entry points need for `rows` tokens. */
uint64_t yvex_b200_moe_workspace_bytes(const yvex_b200_moe_geometry *g, uint64_t rows);

/*
 * Router only: sqrt(softplus(logit)) scoring, bias-corrected top-k with lowest-index tie-break
 * (or the hash table row of the token id), weights = unbiased scores normalised over the
 * selection times the scaling factor. Replaces yvex_moe_route_rows
 * (src/backend/cuda/moe_kernels.cu:180-291); CPU meaning yvex_moe_route_cpu
 * (src/graph/moe.c:520-585). `rows_f32` is the bf16-exact hidden rows [rows x hidden] when the
 * router projection is computed here, otherwise `logits` [rows x experts] is read.
 * selected is [rows x topk] int32, weights [rows x topk] f32.
 */
int yvex_b200_moe_route(const yvex_b200_moe_geometry *g, const yvex_b200_moe_weights *w,
                        const float *rows_f32, const float *logits, const uint32_t *token_ids,
                        uint64_t rows, int32_t *selected, float *weights, float *logits_out,
                        void *workspace, uint64_t workspace_bytes, int *status, void *stream);

/* Ingress rounding of n values (src/graph/moe.c:487-489): rounded_f32 = bf16(x) as f32, rounded_f16 = the same values
 * as fp16 (the rows the expert-parallel dispatch sends and the grouped GEMM reads). Non-finite input sets the status word. */
int yvex_b200_moe_ingress(const float *x, uint64_t n, float *rounded_f32, void *rounded_f16, int *status, void *stream);

/*
 * One MoE FFN layer for a narrow batch (decode): ingress bf16 rounding, router, k routed experts
 * + the shared expert as dequant-fused matvecs with the SwiGLU*weight->bf16 epilogue, per-pair
 * bf16 down outputs summed in rank order, bf16(routed + shared). Replaces the kernel sequence of
 * moe_cuda_graph_enqueue (src/backend/cuda/moe.c:1619-1643) for a layer without the mHC
 * envelope; CPU meaning src/runtime/moe.c:596-632. rows <= 64.
 * x and out are [rows x hidden] f32 on the device.
 */
int yvex_b200_moe_decode(const yvex_b200_moe_geometry *g, const yvex_b200_moe_weights *w,
                         const float *x, const float *logits, const uint32_t *token_ids,
                         uint64_t rows, float *out, int32_t *selected_out, float *weights_out,
                         void *workspace, uint64_t workspace_bytes, int *status, void *stream);
/* The same with the parts of the sum published too (either may be NULL): routed_out = the f32
 * rank-ordered sum of the routed experts' bf16 rows, shared_out = the shared expert's bf16 row, both
 * [rows x hidden] f32 on the device, as the reference's routed_output / shared_output
 * (src/runtime/moe.c:606-637); out = bf16(routed + shared) as before. */
int yvex_b200_moe_decode_parts(const yvex_b200_moe_geometry *g, const yvex_b200_moe_weights *w,
                               const float *x, const float *logits, const uint32_t *token_ids,
                               uint64_t rows, float *out, float *routed_out, float *shared_out,
                               int32_t *selected_out, float *weights_out,
                               void *workspace, uint64_t workspace_bytes, int *status, void *stream);

/*
 * The same layer for a wide batch (prefill / expert-parallel shard): route, expert-major
 * counting sort (permute), grouped dequant GEMM on the tensor cores (gate/up -> SwiGLU*weight
 * -> bf16 -> down -> bf16), rank-ordered unpermute + shared + bf16. No reference counterpart
 * admits more than 62 rows (src/graph/worklist.c:316); semantics per token are those of
 * yvex_b200_moe_decode. `expert_begin/expert_count` restrict routed work to a contiguous
 * expert range (an expert-parallel shard); pairs outside it are left to other ranks.
 */
uint64_t yvex_b200_moe_wide_workspace_bytes(const yvex_b200_moe_geometry *g, uint64_t rows);
/* 1 when yvex_b200_moe_wide runs this layer on the tcgen05 grouped GEMM; 0 when its shapes, its
 * qtypes or a weight pack that does not start on a 16-byte boundary send it to the row kernels
 * (same results, far slower). Lets a caller report or refuse the slow path instead of meeting it. */
int yvex_b200_moe_wide_uses_gemm(const yvex_b200_moe_geometry *g, const yvex_b200_moe_weights *w);
/* Token columns of one grouped-GEMM tile for a weight qtype (0: the qtype has no GEMM decoder). */
uint64_t yvex_b200_moe_wide_tile_columns(unsigned int qtype);
int yvex_b200_moe_wide(const yvex_b200_moe_geometry *g, const yvex_b200_moe_weights *w,
                       const float *x, const float *logits, const uint32_t *token_ids,
                       uint64_t rows, float *out, int32_t *selected_out, float *weights_out,
                       void *workspace, uint64_t workspace_bytes, int *status, void *stream);
/* With routed_out / shared_out as in yvex_b200_moe_decode_parts. */
int yvex_b200_moe_wide_parts(const yvex_b200_moe_geometry *g, const yvex_b200_moe_weights *w,
                             const float *x, const float *logits, const uint32_t *token_ids,
                             uint64_t rows, float *out, float *routed_out, float *shared_out,
                             int32_t *selected_out, float *weights_out,
                             void *workspace, uint64_t workspace_bytes, int *status, void *stream);

/*
 * Expert-parallel building blocks (no reference counterpart: the reference is single-device,
 * src/runtime/moe.c; per-pair semantics are yvex_moe_expert_cpu, src/graph/moe.c:587-622).
 *
 * yvex_b200_moe_expert_rows runs a caller-made pair list on this device's expert shard: pair p is
 * (input row p of rows_f16 [pairs x hidden] - the fp16 image of a bf16-exact row -, expert
 * expert_ids[p] in [0, g->experts) relative to the shard the weight pointers name, or negative
 * for the shared expert, route weight route_weights[p]) and yields y_bf16[p] = bf16(down(bf16(
 * SwiGLU(gate.x, up.x) * weight))) as bf16 bit patterns [pairs x hidden]. g->experts is the
 * number of experts in the shard.
 *
 * yvex_b200_moe_combine is the home rank's unpermute: out[t] = bf16(sum over rank r of
 * y_routed[t*topk + r] in rank order (f32) + y_shared[t]) (src/runtime/moe.c:619-632).
 */
uint64_t yvex_b200_moe_expert_rows_workspace_bytes(const yvex_b200_moe_geometry *g, uint64_t pairs);
int yvex_b200_moe_expert_rows(const yvex_b200_moe_geometry *g, const yvex_b200_moe_weights *w,
                              const void *rows_f16, const int32_t *expert_ids, const float *route_weights,
                              uint64_t pairs, void *y_bf16, void *workspace, uint64_t workspace_bytes,
                              int *status, void *stream);
int yvex_b200_moe_combine(const void *y_routed_bf16, const void *y_shared_bf16, uint64_t tokens,
                          uint64_t topk, uint64_t hidden, float *out, int *status, void *stream);
/*
 * Elementwise steps of the token-local transaction, which runs one expert at a time between
 * yvex_b200_gemv calls like yvex_backend_moe_add_expert (src/backend/cuda/moe.c:673-724). All arrays
 * are device f32 of n elements. _round: out = bf16(x), the ingress rounding of the normalized row
 * (src/graph/moe.c:487-489); _scores: (float)sqrt(softplus(logit)) in double (src/graph/moe.c:497-506);
 * _swiglu: mid = bf16(silu(min(g, limit)) * clamp(u, +-limit) * weight) (src/graph/moe.c:604-616);
 * _accumulate: dst += src (src/runtime/moe.c:620-622); _sum_round: out = bf16(a + b)
 * (src/runtime/moe.c:630-634). Non-finite values set the status word.
 */
int yvex_b200_moe_token_round(const float *x, uint64_t n, float *out, int *status, void *stream);
int yvex_b200_moe_token_scores(const float *logits, uint64_t n, float *scores, int *status, void *stream);
int yvex_b200_moe_token_swiglu(const float *gate, const float *up, uint64_t n, double limit, float weight, float *mid,
                               int *status, void *stream);
int yvex_b200_moe_token_accumulate(const float *src, uint64_t n, float *dst, int *status, void *stream);
int yvex_b200_moe_token_sum_round(const float *a, const float *b, uint64_t n, float *out, int *status, void *stream);
/*
 * The sending side of the expert-parallel dispatch in one call: groups the (token, rank) pairs of
 * `selected` [tokens x topk] by destination rank e / experts_per_rank (stable: ascending pair index
 * within a rank) and writes, in that send order, the fp16 rows (row of pair p = rows_f16[p / topk]),
 * meta[2*pos] = expert id local to its rank and meta[2*pos + 1] = route weight bits; inverse[p] =
 * position of pair p in the send order (what the combine later reads through), send_counts[r] =
 * pairs for rank r (64-bit, the split sizes of the all-to-all-v). No reference counterpart.
 */
uint64_t yvex_b200_ep_dispatch_workspace_bytes(uint64_t pairs, uint64_t world);
int yvex_b200_ep_dispatch(const int32_t *selected, const float *weights, const void *rows_f16, uint64_t tokens,
                          uint64_t topk, uint64_t hidden, uint64_t experts_per_rank, uint64_t world,
                          void *send_rows_f16, int32_t *meta, int32_t *inverse, long long *send_counts,
                          void *workspace, uint64_t workspace_bytes, int *status, void *stream);
/*
 * The same dispatch for an exchange that is pipelined against the expert GEMMs. Each destination
 * rank's experts are cut into `segments` equal ranges, and the pairs are grouped by (segment,
 * destination rank), so that segment 0 of every rank can travel and be computed while segment 1 is
 * still on its way. A row travels as one record of yvex_b200_ep_payload_pitch(hidden) bytes: its
 * hidden fp16 values followed by a 16-byte trailer {int32 expert id local to its rank, f32 route
 * weight, int32 pair index at home, int32 home rank}, so no second message carries the metadata. send_counts has
 * world * segments entries, [segment][rank]. yvex_b200_moe_expert_rows_payload runs such records as
 * a pair list (ids and weights from the trailers; a negative id names the shared expert).
 * yvex_b200_moe_wide_set_cta_limit bounds the CTAs of the persistent grouped GEMM (default: one per
 * SM) so that communication kernels find free SMs beside it; process-wide.
 */
uint64_t yvex_b200_ep_payload_pitch(uint64_t hidden);
int yvex_b200_ep_dispatch_payload(const int32_t *selected, const float *weights, const void *rows_f16, uint64_t tokens,
                                  uint64_t topk, uint64_t hidden, uint64_t experts_per_rank, uint64_t world,
                                  uint64_t rank, uint64_t segments, void *payload, int32_t *inverse, long long *send_counts,
                                  void *workspace, uint64_t workspace_bytes, int *status, void *stream);
int yvex_b200_moe_expert_rows_payload(const yvex_b200_moe_geometry *g, const yvex_b200_moe_weights *w,
                                      const void *payload, uint64_t pairs, void *y_bf16, void *workspace,
                                      uint64_t workspace_bytes, int *status, void *stream);
/*
 * The dispatch without a bulk collective, in two calls around one all-gather of the counts.
 * yvex_b200_ep_dispatch_plan groups the pairs as above (inverse index, send_counts[segments * world]) and
 * leaves the plan in `workspace`. Once every rank knows every rank's counts (counts_all[world][segments *
 * world], device), yvex_b200_ep_dispatch_push (same workspace) writes each payload row straight into the
 * destination rank's receive buffer of its segment: recv_bases[bin] is that buffer's byte address (bin =
 * segment * world + destination; peers' buffers mapped into this address space; plain stores over NVLink,
 * no multicast), rows of one bin ordered by source rank. A row that would land at or past capacity_rows
 * sets status 2 and is not stored. The receiver may read its buffers once every rank's push has finished
 * (any barrier).
 * expert_major = 1 (needs segments == experts_per_rank, i.e. one bin per (local expert, destination), and ONE
 * receive buffer per destination rank: recv_bases[bin] = that rank's buffer for every bin): the bins of a
 * destination follow each other in local-expert order, so its rows arrive already sorted the way the grouped
 * GEMM walks them; yvex_b200_moe_expert_rows_sorted then runs them where they lie (activation tiles fetched
 * with the records' pitch, no count / sort / gather pass), storing the results at their home ranks like
 * yvex_b200_moe_expert_rows_scatter. It refuses gate/up qtypes with a min term (YVEX_ERR_UNSUPPORTED).
 */
int yvex_b200_ep_dispatch_plan(const int32_t *selected, uint64_t tokens, uint64_t topk, uint64_t experts_per_rank, uint64_t world,
                               uint64_t segments, int32_t *inverse, long long *send_counts, void *workspace, uint64_t workspace_bytes,
                               int *status, void *stream);
int yvex_b200_ep_dispatch_push(const int32_t *selected, const float *weights, const void *rows_f16, uint64_t tokens, uint64_t topk,
                               uint64_t hidden, uint64_t experts_per_rank, uint64_t world, uint64_t rank, uint64_t segments,
                               const long long *counts_all, const unsigned long long *recv_bases, uint64_t capacity_rows,
                               int expert_major, void *workspace, uint64_t workspace_bytes, int *status, void *stream);
int yvex_b200_moe_expert_rows_sorted(const yvex_b200_moe_geometry *g, const yvex_b200_moe_weights *w, const void *payload,
                                     uint64_t pairs, const long long *counts_all, uint64_t world, uint64_t rank,
                                     const unsigned long long *home_bases, uint64_t home_pairs, void *workspace,
                                     uint64_t workspace_bytes, int *status, void *stream);
/*
 * The same GEMMs with the return exchange fused into the down projection: the epilogue stores every
 * pair's bf16 row straight into its HOME rank's buffer, at home_bases[home rank] + home pair * hidden * 2
 * (home_bases: device array of `world` byte addresses, this GPU's own buffer and its peers' mapped into
 * this address space; plain stores over NVLink, no multicast). Nothing is returned by a collective: the
 * caller only has to know that every rank's kernel has finished (any barrier) before it sums the rows.
 * A trailer that names a rank >= world or a pair >= home_pairs sets status 2 and its row is dropped.
 */
int yvex_b200_moe_expert_rows_scatter(const yvex_b200_moe_geometry *g, const yvex_b200_moe_weights *w,
                                      const void *payload, uint64_t pairs, const unsigned long long *home_bases,
                                      uint64_t world, uint64_t home_pairs, void *workspace, uint64_t workspace_bytes,
                                      int *status, void *stream);
int yvex_b200_moe_wide_set_cta_limit(int ctas);
/* The same sum with the rows named by index: routed row (t, r) is y_routed[routed_rows[t*topk + r]],
 * the shared row of token t is y_shared[shared_rows[t]]; a NULL index means the identity order.
 * Lets an expert-parallel home rank combine straight from its receive buffer. */
int yvex_b200_moe_combine_indexed(const void *y_routed_bf16, const int32_t *routed_rows, const void *y_shared_bf16,
                                  const int32_t *shared_rows, uint64_t tokens, uint64_t topk, uint64_t hidden,
                                  float *out, int *status, void *stream);

/*
 * Expert worklist of a routed batch: the stable expert-major counting sort of the (row, rank)
 * pairs and its pointer-free summary. Replaces yvex_expert_worklist_build_cuda
 * (src/backend/cuda/moe_kernels.cu:294-397); CPU meaning yvex_expert_worklist_build
 * (src/graph/worklist.c:369-441): buckets ascending by expert id, only populated experts get a
 * bucket, pairs ascending within a bucket, source_rows[i] = pair / topk, destination_rows[i] =
 * pair. The observation has the layout of yvex_expert_worklist_observation
 * (include/yvex/internal/execution_batch.h:126-137) so the host boundary can hand it on as is.
 * Unlike the reference's builder the row count is not limited to 62. Every output pointer is
 * optional; index arrays are int32 on the device. Batches of more than 2048 pairs need
 * yvex_b200_expert_worklist_workspace_bytes() of scratch and run the wide path's own sort
 * kernels; smaller ones take no scratch and one launch.
 */
#define YVEX_B200_WORKLIST_HISTOGRAM_CAP 17u
#define YVEX_B200_WORKLIST_PROVENANCE_COUNT 5u
typedef struct yvex_b200_worklist_observation {
    unsigned int schema_version;
    unsigned long long worklist_count, pair_count, bucket_count;
    unsigned long long maximum_bucket_population;
    unsigned long long tensor_core_eligible_pairs, tensor_core_executed_pairs;
    unsigned long long narrow_pairs, tail_rows;
    unsigned long long width_histogram[YVEX_B200_WORKLIST_HISTOGRAM_CAP];
    unsigned long long population_histogram[YVEX_B200_WORKLIST_HISTOGRAM_CAP];
    unsigned long long provenance_counts[YVEX_B200_WORKLIST_PROVENANCE_COUNT];
} yvex_b200_worklist_observation;
uint64_t yvex_b200_expert_worklist_workspace_bytes(uint64_t pairs, uint64_t experts);
int yvex_b200_expert_worklist(const int32_t *selected, uint64_t rows, uint64_t topk, uint64_t experts,
                              uint64_t tensor_core_minimum, uint64_t admitted_width, unsigned int provenance,
                              int32_t *source_pairs, int32_t *source_rows, int32_t *destination_rows,
                              int32_t *expert_ids, int32_t *bucket_offsets, int32_t *bucket_populations,
                              yvex_b200_worklist_observation *observation, void *workspace,
                              uint64_t workspace_bytes, int *status, void *stream);

/*
 * Self-test of the bounded device waits: one CTA waits on an mbarrier that nothing arrives on,
 * with a limit of `limit_ns` nanoseconds of the device clock. The wait must run out: the kernel
 * then raises status 3 (YVEX_B200_STATUS_TIMEOUT), writes the time it waited to *elapsed_ns
 * (device memory, optional) and returns; no copy or tensor-core work is in flight, the context
 * stays usable. No counterpart in the reference, whose kernels do not wait on one another.
 */
int yvex_b200_selftest_bounded_wait(uint64_t limit_ns, uint64_t *elapsed_ns, int *status, void *stream);

/*
 * mHC envelope of the MoE FFN: the layer's rows carry `streams` residual streams
 * (expanded width = streams * hidden). yvex_b200_mhc_prepare is yvex_moe_ffn_prepare_cpu
 * (src/graph/moe.c:446-495: mixing projection, yvex_attention_mhc_pre of
 * src/graph/numeric.c:752-824, RMSNorm * weight, bf16 rounding) and the device twin of
 * yvex_residual_mhc_pre + yvex_attention_weighted_norm (src/backend/cuda/kernels.cu:1243-1388,
 * 867-911): expanded [rows x streams*hidden] f32 -> normalized [rows x hidden] (the FFN input),
 * post [rows x streams], combination [rows x streams*streams]. yvex_b200_mhc_post is
 * yvex_attention_mhc_post (src/graph/numeric.c:826-875; CUDA twin yvex_residual_mhc_post,
 * src/backend/cuda/kernels.cu:1389-1421): core [rows x hidden] -> out [rows x streams*hidden].
 * Coefficients are device F32 arrays: mhc_fn [(streams+2)*streams x streams*hidden], scale [3],
 * base [(streams+2)*streams], norm [hidden]. Limits of the reference: (streams+2)*streams <= 64,
 * hidden <= 16384.
 */
typedef struct yvex_b200_mhc {
    uint64_t hidden, streams, sinkhorn_iterations;
    double rms_epsilon, mhc_epsilon, post_multiplier;
    const float *mhc_fn, *scale, *base, *norm;
} yvex_b200_mhc;
uint64_t yvex_b200_mhc_workspace_bytes(uint64_t streams, uint64_t rows);
int yvex_b200_mhc_prepare(const yvex_b200_mhc *m, const float *expanded, uint64_t rows, float *normalized,
                          float *post, float *combination, void *workspace, uint64_t workspace_bytes,
                          int *status, void *stream);
int yvex_b200_mhc_post(const yvex_b200_mhc *m, const float *core, const float *expanded, const float *post,
                       const float *combination, uint64_t rows, float *out, int *status, void *stream);

/*
 * Online-softmax causal GQA attention at decode: one query position per session against a bf16
 * KV cache, f32 accumulation and output. q [sessions][q_heads][head_dim] bf16, k/v
 * [sessions][kv_heads][context][head_dim] bf16, out [sessions][q_heads][head_dim] f32; keys
 * 0..position are visible. Replaces the online-softmax core of yvex_attention_reduce_native
 * (src/backend/cuda/attention_kernels.cu:259-406) and yvex_gqa_causal_f32
 * (src/backend/cuda/transformer_kernels.cu:85-145); CPU meaning: cpu_op_attention
 * (src/backend/cpu.c:319-411) per (session, q head). scratch holds the split-KV partials.
 */
uint64_t yvex_b200_attention_workspace_bytes(uint64_t sessions, uint64_t q_heads,
                                             uint64_t kv_heads, uint64_t head_dim,
                                             uint64_t context);
int yvex_b200_attention_gqa_decode(const void *q_bf16, const void *k_bf16, const void *v_bf16,
                                   uint64_t sessions, uint64_t q_heads, uint64_t kv_heads,
                                   uint64_t head_dim, uint64_t context, uint64_t position,
                                   float scale, float *out, void *workspace,
                                   uint64_t workspace_bytes, int *status, void *stream);

/*
 * The same operation for callers that can pass no workspace and must not cause a device-memory
 * allocation (a runtime whose device bytes are all planned up front, or a latency-critical path
 * that may not enter the allocator). This entry point has no counterpart in the reference. The
 * split-KV partials live in one fixed 8 MiB device array per device
 * (yvex_b200_attention_static_scratch_bytes()); a problem whose partials do not fit is refused
 * with YVEX_ERR_BOUNDS (-7) before any launch. The first call on a device resolves the array's
 * address and should be made during start-up, before any stream capture; the array is that of the
 * device current in the calling thread, and `stream` must belong to that device; calls that overlap
 * in time on one device race on the array and must be serialised by the caller. Results are
 * identical to yvex_b200_attention_gqa_decode.
 */
uint64_t yvex_b200_attention_static_scratch_bytes(void);
int yvex_b200_attention_gqa_decode_static(const void *q_bf16, const void *k_bf16, const void *v_bf16,
                                          uint64_t sessions, uint64_t q_heads, uint64_t kv_heads,
                                          uint64_t head_dim, uint64_t context, uint64_t position,
                                          float scale, float *out, int *status, void *stream);

/*
 * Single-head f32 attention, the public op of the reference vtable (op_attention,
 * src/backend/cpu.c:319-411, src/backend/cuda/kernels.cu:362-435): q [d], keys/values
 * [seq_len x d] f32, scores/probabilities [seq_len] written like the reference does.
 */
int yvex_b200_attention_f32(const float *q, const float *keys, const float *values,
                            uint64_t seq_len, uint64_t head_dim, uint64_t position, float scale,
                            int causal, float *scores, float *probabilities, float *out,
                            int *status, void *stream);

/*
 * Sink reducer of the graph attention op: every query head of one token against one row set that is key
 * and value at once and is shared by all heads (reduce_head / reduce_visit_row, src/graph/core.c:428-465,
 * :318-345). query [heads x head_dim], rows [row_count x head_dim], sinks [heads], out [heads x head_dim],
 * all f32 on the device. Scores are f64 dot products times scale; the head's sink is the initial maximum
 * and seeds the denominator with exp(sink - max) without contributing a value; out = sum p * row /
 * denominator, rounded to bf16 when round_bf16 is set (the compute contract's rounding). row_count may be
 * 0 (the output is then zero: only the sink has weight). The rotary step the reference applies to the
 * result afterwards is not part of this entry. head_dim <= 1024.
 */
int yvex_b200_attention_sink(const float *query, const float *rows, const float *sinks, uint64_t heads, uint64_t row_count,
                             uint64_t head_dim, double scale, int round_bf16, float *out, int *status, void *stream);

#ifdef __cplusplus
}
#endif
#endif
