/*
 * The MoE operation table of the host boundary: workspace_required / execute_rows / complete_rows
 * with the reference's contract (include/yvex/internal/moe.h:277-297, src/backend/cuda/moe.c:1826-1966),
 * plus the unbounded-width extension. The layer itself runs in the device layer
 * (yvex_b200_moe_decode for <= 62 rows, yvex_b200_moe_wide beyond). At the end of the file: the
 * token-local transaction (begin / add_expert / finish / close), one expert per call.
 *
 * Two row shapes. Without the envelope (residual_streams <= 1, expanded_width == hidden_width) the
 * input rows are the normalized hidden rows, rounded to bf16 at ingress like the reference's
 * normalized row (src/graph/moe.c:487-489). With the mHC envelope (residual_streams > 1) rows are
 * the expanded residual rows on both sides, as in the reference's execute_rows
 * (src/backend/cuda/moe.c:1381-1543): prepare (mixing projection, gates, Sinkhorn, collapse,
 * RMSNorm; src/graph/moe.c:446-495) -> layer -> post (src/graph/numeric.c:826-875). The envelope's
 * coefficient tensors must be resident F32; anything else is refused, never skipped.
 */
#define _POSIX_C_SOURCE 200809L
#include "backend_private.h"

#include <stdlib.h>
#include <string.h>
#include <time.h>

/* Row chunks of the wide entry's copy pipeline. Rows are independent, so a batch of host rows may
 * run as consecutive row ranges: while range i is computed, range i + 1 is on its way in and range
 * i - 1 on its way out. A range still has to fill the grouped GEMM's token tiles, so the count
 * follows the average pairs per expert (about 160 per range, at most YVEX_MOE_MAX_CHUNKS). */
static unsigned long long wide_chunks(const yvex_b200_moe_geometry *g, unsigned long long rows) {
    const unsigned long long per_expert = rows * g->topk / (g->experts ? g->experts : 1ull), n = per_expert / 160ull;
    return n < 1ull ? 1ull : n > (unsigned long long)YVEX_MOE_MAX_CHUNKS ? (unsigned long long)YVEX_MOE_MAX_CHUNKS : n;
}

#define YVEX_MOE_NARROW_MAX_ROWS 62ull       /* src/graph/worklist.c:316, src/backend/cuda/moe.c:1840-1843 */

static int family_admitted(const char *family) {
    return !family || !strcmp(family, YVEX_MOE_KERNEL_SM100_DEQUANT_GEMV) || !strcmp(family, YVEX_MOE_KERNEL_SM100_TCGEN05_EXPERT);
}

static int plan_geometry(const yvex_moe_layer_plan *layer, const yvex_moe_layer_job *job, yvex_b200_moe_geometry *g) {
    memset(g, 0, sizeof(*g));
    g->hidden = layer->hidden_width;
    g->experts = layer->routed_experts;
    g->topk = layer->experts_per_token;
    g->inter = layer->expert_intermediate_width;
    g->shared_inter = layer->shared_intermediate_width ? layer->shared_intermediate_width : layer->expert_intermediate_width;
    g->scaling = layer->routed_scaling_factor;
    g->limit = layer->activation_limit;
    g->normalize = layer->normalize_topk_probabilities;
    g->router_class = layer->router_class == YVEX_MOE_ROUTER_LEARNED_HIDDEN_STATE ? 1 : 0;
    g->hash_rows = layer->hash_table_rows;
    if (job) {
        g->gate_qtype = job->weights[YVEX_MOE_WEIGHT_ROUTED_GATE].qtype;
        g->up_qtype = job->weights[YVEX_MOE_WEIGHT_ROUTED_UP].qtype;
        g->down_qtype = job->weights[YVEX_MOE_WEIGHT_ROUTED_DOWN].qtype;
        g->hash_stored_rows = job->weights[YVEX_MOE_WEIGHT_ROUTER_TABLE].row_count;
    } else {
        g->gate_qtype = g->up_qtype = g->down_qtype = 16u;   /* sizes do not depend on the qtype */
    }
    return 1;
}

static unsigned long long align256(unsigned long long v) { return (v + 255ull) & ~255ull; }

static unsigned long long envelope_streams(const yvex_moe_layer_plan *layer) {
    return layer->residual_streams > 1ull ? layer->residual_streams : 1ull;
}

/* Rows in and out are `streams` times wider with the envelope, which also needs the normalized and
 * combined hidden rows, the gates and the device layer's own scratch. */
static unsigned long long staging_bytes(const yvex_b200_moe_geometry *g, unsigned long long rows, unsigned long long streams) {
    /* rows in and out, logits, selection, token ids, and the routed / shared parts of the sum */
    unsigned long long bytes = 2ull * align256(rows * g->hidden * streams * 4ull) + align256(rows * g->experts * 4ull) +
                               2ull * align256(rows * g->topk * 4ull) + align256(rows * 4ull) + 2ull * align256(rows * g->hidden * 4ull) +
                               256ull;
    if (streams > 1ull) {
        const unsigned long long mix_rows = (streams + 2ull) * streams;
        bytes += 2ull * align256(rows * g->hidden * 4ull) + align256(rows * streams * 4ull) + align256(rows * streams * streams * 4ull) +
                 align256(yvex_b200_mhc_workspace_bytes(streams, rows));
        /* F32 images of BF16 coefficient tensors (norm, mixing function, base, scale) */
        bytes += align256(g->hidden * 4ull) + align256(mix_rows * streams * g->hidden * 4ull) + align256(mix_rows * 4ull) + align256(12ull);
    }
    return bytes;
}

/* Scratch of the token-local transaction (one row, one expert at a time). */
static unsigned long long token_inter(const yvex_b200_moe_geometry *g) { return g->inter > g->shared_inter ? g->inter : g->shared_inter; }
static unsigned long long token_bytes(const yvex_b200_moe_geometry *g, unsigned long long streams) {
    unsigned long long bytes = 2ull * align256(streams * g->hidden * 4ull) + 5ull * align256(g->hidden * 4ull) + 3ull * align256(token_inter(g) * 4ull) +
                               2ull * align256(g->experts * 4ull) + 2ull * align256(g->topk * 4ull) + 512ull;
    if (streams > 1ull) {
        const unsigned long long mix_rows = (streams + 2ull) * streams;
        bytes += align256(streams * 4ull) + align256(streams * streams * 4ull) + align256(yvex_b200_mhc_workspace_bytes(streams, 1ull)) +
                 align256(g->hidden * 4ull) + align256(mix_rows * streams * g->hidden * 4ull) + align256(mix_rows * 4ull) + align256(12ull);
    }
    return bytes;
}

static int workspace_for(const yvex_moe_layer_plan *layer, unsigned long long rows, int wide, unsigned long long *bytes, yvex_error *err) {
    yvex_b200_moe_geometry g;
    if (bytes) *bytes = 0;
    if (!layer || !bytes || !rows) return yvex_refuse(err, YVEX_ERR_INVALID_ARG, "moe.workspace_required", "layer, rows and result are required");
    if (!wide && rows > YVEX_MOE_NARROW_MAX_ROWS)
        return yvex_refuse(err, YVEX_ERR_UNSUPPORTED, "moe.workspace_required", "execute_rows admits at most 62 rows; use the wide entry");
    plan_geometry(layer, NULL, &g);
    {
        unsigned long long kernel = wide ? yvex_b200_moe_wide_workspace_bytes(&g, rows) : yvex_b200_moe_workspace_bytes(&g, rows);
        const unsigned long long list = yvex_b200_expert_worklist_workspace_bytes(rows * g.topk, g.experts);
        *bytes = staging_bytes(&g, rows, envelope_streams(layer)) + (kernel > list ? kernel : list);
        if (*bytes < token_bytes(&g, envelope_streams(layer))) *bytes = token_bytes(&g, envelope_streams(layer));
    }
    yvex_error_clear(err);
    return YVEX_OK;
}

static int moe_workspace_required(const yvex_moe_layer_plan *layer, unsigned long long rows, unsigned long long *bytes, yvex_error *err) {
    return workspace_for(layer, rows, 0, bytes, err);
}

static int moe_workspace_required_wide(const yvex_moe_layer_plan *layer, unsigned long long rows, unsigned long long *bytes, yvex_error *err) {
    return workspace_for(layer, rows, 1, bytes, err);
}

static int derived_plan(const void *decision, unsigned long long *storage_bytes, yvex_error *err) {
    (void)decision;
    if (storage_bytes) *storage_bytes = 0;
    return yvex_refuse(err, YVEX_ERR_UNSUPPORTED, "moe.derived_layout_plan", "this backend executes the canonical row layout only");
}

static int derived_build(const void *decision, const unsigned char *canonical, unsigned long long canonical_bytes,
                         unsigned char *derived, unsigned long long storage_bytes, yvex_error *err) {
    (void)decision; (void)canonical; (void)canonical_bytes; (void)derived; (void)storage_bytes;
    return yvex_refuse(err, YVEX_ERR_UNSUPPORTED, "moe.derived_layout_build", "this backend executes the canonical row layout only");
}

/* Resolves one weight view to its device address; optional slots resolve to 0. */
static int resolve_view(const yvex_backend *backend, const yvex_moe_weight_view *v, int required, const void **out) {
    unsigned long long address = 0;
    *out = NULL;
    if (v->device_address) { *out = (const void *)(uintptr_t)v->device_address; return 1; }
    if (!v->encoded || !v->encoded_bytes) return required ? 0 : 1;
    if (yvex_backend_resident_resolve(backend, v->encoded, v->encoded_bytes, &address) != YVEX_BACKEND_RESIDENT_HIT) return 0;
    *out = (const void *)(uintptr_t)address;
    return 1;
}

static int view_consistent(const yvex_moe_weight_view *v, unsigned long long rows, unsigned long long width) {
    unsigned int be = 0, bb = 0;
    if (!yvex_b200_qtype_geometry(v->qtype, &be, &bb) || !be) return 0;
    return v->row_count == rows && v->row_width == width && width % be == 0 && v->row_bytes == width / be * bb &&
           v->encoded_bytes == rows * v->row_bytes;
}

static int status_error(int code, yvex_error *err) {
    if (!code) return YVEX_OK;
    if (code == YVEX_B200_STATUS_TIMEOUT) return yvex_refuse(err, YVEX_ERR_TIMEOUT, "cuda.moe", "a bounded device wait expired");
    return yvex_refuse(err, YVEX_ERR_BACKEND, "cuda.moe", "CUDA MoE kernel reported invalid or non-finite numerics");
}

/* What the kernels of one row batch read and write: everything the enqueue below needs, and (as plain words) the
 * identity of a launch graph that replays it. */
typedef struct {
    yvex_backend *backend;
    const yvex_moe_layer_job *job;
    yvex_b200_moe_geometry g;
    yvex_b200_moe_weights w;
    yvex_b200_mhc mhc;
    unsigned long long streams, rows, mhc_ws, kernel_ws, tensor_path, coeff_count[4];
    int wide;
    unsigned int provenance;
    const void *coeff_addr[4];
    unsigned int coeff_qtype[4];
    const float *dev_in, *dev_logits;
    float *dev_out;
    const uint32_t *ids;
    unsigned char *ws_norm, *ws_core, *ws_post, *ws_comb, *ws_mhc, *ws_coeff[4], *ws_routed, *ws_shared, *ws_sel, *ws_wts, *ws_kernel;
    yvex_expert_worklist_observation *dev_obs;
} rows_run;

/* The layer of a batch that is not pipelined: envelope prepare, the MoE layer, envelope post. */
static int rows_layer(rows_run *r, const char **message) {
    yvex_backend *backend = r->backend;
    const float *layer_in = r->dev_in;
    float *layer_out = r->dev_out;
    int rc;
    if (r->streams > 1ull) {
        const float **slot_ptr[4] = {&r->mhc.norm, &r->mhc.mhc_fn, &r->mhc.base, &r->mhc.scale};
        *message = "device layer refused an mHC coefficient tensor";
        for (int i = 0; i < 4; ++i) {
            if (r->coeff_qtype[i] != 30u) continue;
            rc = yvex_b200_dequant_rows(30u, r->coeff_addr[i], 1ull, r->coeff_count[i], r->coeff_count[i] * 2ull, (float *)r->ws_coeff[i],
                                        backend->status_word, backend->stream);
            if (rc != YVEX_OK) return rc;
            *slot_ptr[i] = (const float *)r->ws_coeff[i];
        }
        *message = "device layer refused the mHC envelope geometry";
        rc = yvex_b200_mhc_prepare(&r->mhc, r->dev_in, r->rows, (float *)r->ws_norm, (float *)r->ws_post, (float *)r->ws_comb, r->ws_mhc,
                                   r->mhc_ws, backend->status_word, backend->stream);
        if (rc != YVEX_OK) return rc;
        layer_in = (const float *)r->ws_norm;
        layer_out = (float *)r->ws_core;
    }
    *message = "device layer refused the MoE layer geometry";
    rc = (r->wide ? yvex_b200_moe_wide_parts : yvex_b200_moe_decode_parts)(
        &r->g, &r->w, layer_in, r->dev_logits, r->ids, r->rows, layer_out, (float *)r->ws_routed, (float *)r->ws_shared, (int32_t *)r->ws_sel,
        (float *)r->ws_wts, r->ws_kernel, r->kernel_ws, backend->status_word, backend->stream);
    if (rc != YVEX_OK) return rc;
    if (r->streams > 1ull) {
        *message = "device layer refused the mHC envelope geometry";
        rc = yvex_b200_mhc_post(&r->mhc, (const float *)r->ws_core, r->dev_in, (const float *)r->ws_post, (const float *)r->ws_comb, r->rows,
                                r->dev_out, backend->status_word, backend->stream);
    }
    return rc;
}

/* The worklist summary of the batch (src/backend/cuda/moe.c:1710-1726), built on the device from the
 * router's selection. The wide path sends every pair through the tensor-core GEMM tiles; the narrow
 * path has no admission threshold, which the reference's summary counts as narrow pairs. */
static int rows_worklist(rows_run *r, const char **message) {
    *message = "device layer refused the expert worklist geometry";
    return yvex_b200_expert_worklist((const int32_t *)r->ws_sel, r->rows, r->g.topk, r->g.experts, r->wide && r->tensor_path ? 1ull : 0ull,
                                     r->wide && r->tensor_path ? yvex_b200_moe_wide_tile_columns(r->g.gate_qtype) : 1ull, r->provenance, NULL,
                                     NULL, NULL, NULL, NULL, NULL, r->dev_obs, r->ws_kernel, r->kernel_ws, r->backend->status_word,
                                     r->backend->stream);
}

/* ---- launch graphs of the narrow entry ---------------------------------------------------------------- */

void yvex_moe_graphs_release(yvex_backend *backend) {
    for (int i = 0; i < YVEX_MOE_GRAPH_SLOTS; ++i) {
        if (backend->moe_graphs[i].exec) cudaGraphExecDestroy(backend->moe_graphs[i].exec);
        memset(&backend->moe_graphs[i], 0, sizeof(backend->moe_graphs[i]));
    }
}

static unsigned long long bits_of(double v) { unsigned long long u; memcpy(&u, &v, sizeof(u)); return u; }

/* Every value a captured kernel argument was computed from. Two batches with equal keys enqueue identical launches. */
static void rows_key(const rows_run *r, int want_parts, unsigned long long *key) {
    const unsigned long long words[] = {
        r->rows, r->streams, (unsigned long long)want_parts, r->provenance, r->g.hidden, r->g.experts, r->g.topk, r->g.inter, r->g.shared_inter,
        r->g.gate_qtype, r->g.up_qtype, r->g.down_qtype, (unsigned long long)r->g.router_class, (unsigned long long)r->g.normalize, r->g.hash_rows,
        r->g.hash_stored_rows, bits_of(r->g.scaling), bits_of(r->g.limit), (uintptr_t)r->w.router, (uintptr_t)r->w.bias, (uintptr_t)r->w.hash_table,
        (uintptr_t)r->w.gate, (uintptr_t)r->w.up, (uintptr_t)r->w.down, (uintptr_t)r->w.shared_gate, (uintptr_t)r->w.shared_up,
        (uintptr_t)r->w.shared_down, (uintptr_t)r->coeff_addr[0], (uintptr_t)r->coeff_addr[1], (uintptr_t)r->coeff_addr[2],
        (uintptr_t)r->coeff_addr[3], r->coeff_qtype[0], r->coeff_qtype[1], r->coeff_qtype[2], r->coeff_qtype[3], r->mhc.sinkhorn_iterations,
        bits_of(r->mhc.rms_epsilon), bits_of(r->mhc.mhc_epsilon), bits_of(r->mhc.post_multiplier), (uintptr_t)r->dev_in, (uintptr_t)r->dev_out,
        (uintptr_t)r->dev_logits, (uintptr_t)r->ids, (uintptr_t)r->backend->workspace->data, r->backend->workspace->bytes};
    _Static_assert(sizeof(words) / sizeof(words[0]) <= YVEX_MOE_GRAPH_KEY_WORDS, "graph key is too small");
    memset(key, 0, YVEX_MOE_GRAPH_KEY_WORDS * sizeof(*key));
    memcpy(key, words, sizeof(words));
}

static yvex_moe_graph_slot *graph_slot(yvex_backend *backend, const unsigned long long *key) {
    yvex_moe_graph_slot *oldest = &backend->moe_graphs[0];
    for (int i = 0; i < YVEX_MOE_GRAPH_SLOTS; ++i) {
        yvex_moe_graph_slot *s = &backend->moe_graphs[i];
        if (s->seen && !memcmp(s->key, key, sizeof(s->key))) { s->stamp = ++backend->moe_graph_stamp; return s; }
        if (s->stamp < oldest->stamp) oldest = s;
    }
    if (oldest->exec) cudaGraphExecDestroy(oldest->exec);           /* least recently used; the stream is idle between calls */
    memset(oldest, 0, sizeof(*oldest));
    memcpy(oldest->key, key, sizeof(oldest->key));
    oldest->stamp = ++backend->moe_graph_stamp;
    return oldest;
}

/* Enqueues the batch's kernels: eagerly the first time a combination is seen, captured into a launch graph and launched
 * the second time, replayed from then on. Returns the device layer's code; *launches = kernels enqueued or replayed. */
static int rows_enqueue_narrow(rows_run *r, int want_parts, yvex_moe_row_batch_result *result, unsigned long long *launches, const char **message) {
    yvex_backend *backend = r->backend;
    unsigned long long key[YVEX_MOE_GRAPH_KEY_WORDS], before = yvex_b200_launch_count();
    yvex_moe_graph_slot *slot = NULL;
    cudaGraph_t graph = NULL;
    int rc;
    if (!yvex_test_seam("YVEX_B200_MOE_GRAPH", "off")) {
        rows_key(r, want_parts, key);
        slot = graph_slot(backend, key);
    }
    if (slot && slot->seen == 2) {
        *message = "launch graph replay failed";
        if (cudaGraphLaunch(slot->exec, backend->stream) != cudaSuccess) return YVEX_ERR_BACKEND;
        *launches = slot->launches;
        result->graph_launches = result->graph_replays = 1ull;
        return YVEX_OK;
    }
    if (slot && slot->seen == 1 && cudaStreamBeginCapture(backend->stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess) {
        rc = rows_layer(r, message);
        if (rc == YVEX_OK) rc = rows_worklist(r, message);
        if (cudaStreamEndCapture(backend->stream, &graph) != cudaSuccess || !graph) {
            cudaGetLastError();
            if (graph) cudaGraphDestroy(graph);
            graph = NULL;
        }
        if (rc != YVEX_OK) {                                    /* a refusal while capturing: nothing was enqueued */
            if (graph) cudaGraphDestroy(graph);
            return rc;
        }
        if (graph && cudaGraphInstantiate(&slot->exec, graph, 0ull) == cudaSuccess) {
            cudaGraphDestroy(graph);
            slot->launches = yvex_b200_launch_count() - before;
            slot->seen = 2;
            *message = "launch graph replay failed";
            if (cudaGraphLaunch(slot->exec, backend->stream) != cudaSuccess) return YVEX_ERR_BACKEND;
            *launches = slot->launches;
            result->graph_launches = result->graph_replays = result->graph_captures = 1ull;
            return YVEX_OK;
        }
        if (graph) cudaGraphDestroy(graph);
        cudaGetLastError();
        slot->exec = NULL;
        slot->seen = -1;                                        /* this combination stays eager */
        before = yvex_b200_launch_count();
    }
    rc = rows_layer(r, message);
    if (rc == YVEX_OK) rc = rows_worklist(r, message);
    if (rc == YVEX_OK && slot && slot->seen == 0) slot->seen = 1;
    *launches = yvex_b200_launch_count() - before;
    return rc;
}

static int moe_execute(yvex_backend *backend, const yvex_moe_layer_job *job, const yvex_moe_row_batch *batch,
                       const yvex_moe_row_batch_output *output, yvex_moe_row_batch_result *result, yvex_error *err, int wide) {
    const char *where = wide ? "cuda.moe.execute_rows_wide" : "cuda.moe.execute_rows";
    const yvex_moe_layer_plan *layer = job ? job->layer : NULL;
    yvex_b200_moe_geometry g;
    yvex_b200_moe_weights w;
    yvex_b200_mhc mhc;
    unsigned long long rows, cursor = 0, need, kernel_ws, launches0, in_bytes, hid_bytes, sel_count, streams, mhc_ws = 0;
    unsigned long long chunks = 1ull, tensor_path, list_ws;
    const float *host_logits = NULL;
    const yvex_device_tensor *tensor_logits = NULL;
    unsigned char *ws_routed = NULL, *ws_shared = NULL;
    int want_parts;
    yvex_expert_worklist_observation *dev_obs, *host_obs;
    unsigned char *ws_in, *ws_out, *ws_logits, *ws_sel, *ws_wts, *ws_ids, *ws_kernel;
    unsigned char *ws_norm = NULL, *ws_core = NULL, *ws_post = NULL, *ws_comb = NULL, *ws_mhc = NULL, *ws_coeff[4] = {NULL, NULL, NULL, NULL};
    unsigned long long coeff_count[4] = {0, 0, 0, 0};
    static const int coeff[4] = {YVEX_MOE_WEIGHT_FFN_NORM, YVEX_MOE_WEIGHT_MHC_FUNCTION, YVEX_MOE_WEIGHT_MHC_BASE, YVEX_MOE_WEIGHT_MHC_SCALE};
    const float *dev_in, *dev_logits = NULL;
    float *dev_out;
    int rc, code, defer, slot, pipelined;
    rows_run run;
    const char *refusal = "device layer refused the MoE layer geometry";
    unsigned long long graph_kernel_launches = ~0ull;
    static const int required[YVEX_MOE_WEIGHT_COUNT] = {0, 0, 0, 0, 0, 0, 0, 1, 1, 1, 1, 1, 1};
    const void *addr[YVEX_MOE_WEIGHT_COUNT];

    if (result) memset(result, 0, sizeof(*result));
    if (!job || !layer || !batch || !result) return yvex_refuse(err, YVEX_ERR_INVALID_ARG, where, "job, layer, batch and result are required");
    rc = yvex_backend_admit(backend, where, err);
    if (rc != YVEX_OK) return rc;
    if (backend->pending_slot) return yvex_refuse(err, YVEX_ERR_STATE, where, "a deferred MoE completion is still pending");
    /* host-side launch-failure seam (src/backend/cuda/qtype.c:625-661, src/backend/cuda/capability.c:611-629) */
    if (yvex_test_seam("YVEX_TEST_CUDA_LAUNCH_FAILURE", "moe-rows")) return yvex_backend_fail(backend, where, err);
    if (batch->schema_version == YVEX_MOE_ROW_BATCH_SCHEMA_B200_LOGITS) {
        host_logits = ((const yvex_moe_row_batch_logits *)batch)->router_logits;
        tensor_logits = ((const yvex_moe_row_batch_logits *)batch)->device_router_logits;
    } else if (batch->schema_version != YVEX_MOE_ROW_BATCH_SCHEMA_V1) {
        return yvex_refuse(err, YVEX_ERR_INVALID_ARG, where, "row batch schema is not one this backend reads");
    }
    if (job->evidence_level == 3 || (job->eager_execution != 0 && job->eager_execution != 1))       /* src/backend/cuda/moe.c:1028-1030 */
        return yvex_refuse(err, YVEX_ERR_INVALID_ARG, where, "full-evidence or malformed eager execution is not a device-native batch");
    rows = batch->row_count;
    if (!rows) return yvex_refuse(err, YVEX_ERR_INVALID_ARG, where, "row batch is empty");
    if (!wide && rows > YVEX_MOE_NARROW_MAX_ROWS)
        return yvex_refuse(err, YVEX_ERR_UNSUPPORTED, where, "row count is outside the admitted widths of execute_rows");
    streams = envelope_streams(layer);
    if (layer->expanded_width && layer->expanded_width != streams * layer->hidden_width)
        return yvex_refuse(err, YVEX_ERR_FORMAT, where, "expanded width is not residual streams x hidden width");
    if (streams > 1ull && layer->mhc_mixing_rows != (streams + 2ull) * streams)
        return yvex_refuse(err, YVEX_ERR_FORMAT, where, "mHC mixing rows must be (streams + 2) x streams");
    if (batch->row_width != streams * layer->hidden_width || (batch->row_stride && batch->row_stride != batch->row_width))
        return yvex_refuse(err, YVEX_ERR_FORMAT, where, "row batch geometry does not match the layer's row width");
    if (!batch->device_rows == !batch->expanded_rows)
        return yvex_refuse(err, YVEX_ERR_INVALID_ARG, where, "exactly one of device rows and host rows is required");
    plan_geometry(layer, job, &g);
    for (slot = YVEX_MOE_WEIGHT_ROUTED_GATE; slot < YVEX_MOE_WEIGHT_COUNT; ++slot) {
        if (!family_admitted(job->weights[slot].kernel_family))
            return yvex_refuse(err, YVEX_ERR_UNSUPPORTED, where, "kernel family is not one this backend executes");
        if (job->weights[slot].layout == YVEX_EXECUTION_LAYOUT_DERIVED_BACKEND)
            return yvex_refuse(err, YVEX_ERR_UNSUPPORTED, where, "this backend offers no derived weight layout");
        if (!yvex_b200_qtype_supported(job->weights[slot].qtype))
            return yvex_refuse(err, YVEX_ERR_UNSUPPORTED, where, "expert qtype has no device decoder in this backend");
    }
    if (job->weights[YVEX_MOE_WEIGHT_SHARED_GATE].qtype != g.gate_qtype || job->weights[YVEX_MOE_WEIGHT_SHARED_UP].qtype != g.up_qtype ||
        job->weights[YVEX_MOE_WEIGHT_SHARED_DOWN].qtype != g.down_qtype)
        return yvex_refuse(err, YVEX_ERR_UNSUPPORTED, where, "shared and routed experts must share their qtypes");
    if (!view_consistent(&job->weights[YVEX_MOE_WEIGHT_ROUTED_GATE], g.experts * g.inter, g.hidden) ||
        !view_consistent(&job->weights[YVEX_MOE_WEIGHT_ROUTED_UP], g.experts * g.inter, g.hidden) ||
        !view_consistent(&job->weights[YVEX_MOE_WEIGHT_ROUTED_DOWN], g.experts * g.hidden, g.inter) ||
        !view_consistent(&job->weights[YVEX_MOE_WEIGHT_SHARED_GATE], g.shared_inter, g.hidden) ||
        !view_consistent(&job->weights[YVEX_MOE_WEIGHT_SHARED_UP], g.shared_inter, g.hidden) ||
        !view_consistent(&job->weights[YVEX_MOE_WEIGHT_SHARED_DOWN], g.hidden, g.shared_inter))
        return yvex_refuse(err, YVEX_ERR_FORMAT, where, "expert weight views are inconsistent with the layer geometry");
    if (job->cancel_requested && job->cancel_requested(job->cancel_context))
        return yvex_refuse(err, YVEX_ERR_CANCELLED, where, "MoE execution was cancelled");
    for (slot = 0; slot < YVEX_MOE_WEIGHT_COUNT; ++slot)
        if (!resolve_view(backend, &job->weights[slot], required[slot], &addr[slot]))
            return yvex_refuse(err, YVEX_ERR_STATE, where, "MoE weights are not resident on this backend");
    memset(&w, 0, sizeof(w));
    w.router = (const float *)addr[YVEX_MOE_WEIGHT_ROUTER];
    w.bias = (const float *)addr[YVEX_MOE_WEIGHT_ROUTER_BIAS];
    w.hash_table = (const int32_t *)addr[YVEX_MOE_WEIGHT_ROUTER_TABLE];
    w.gate = addr[YVEX_MOE_WEIGHT_ROUTED_GATE]; w.up = addr[YVEX_MOE_WEIGHT_ROUTED_UP]; w.down = addr[YVEX_MOE_WEIGHT_ROUTED_DOWN];
    w.shared_gate = addr[YVEX_MOE_WEIGHT_SHARED_GATE]; w.shared_up = addr[YVEX_MOE_WEIGHT_SHARED_UP];
    w.shared_down = addr[YVEX_MOE_WEIGHT_SHARED_DOWN];
    if (w.router && (job->weights[YVEX_MOE_WEIGHT_ROUTER].qtype != 0u ||
                     job->weights[YVEX_MOE_WEIGHT_ROUTER].encoded_bytes != g.experts * g.hidden * 4ull))
        return yvex_refuse(err, YVEX_ERR_UNSUPPORTED, where, "router weights must be F32 [experts x hidden]");
    if (!w.router && !host_logits && !tensor_logits)
        return yvex_refuse(err, YVEX_ERR_INVALID_ARG, where, "either resident router weights or router logits are required");
    if (g.router_class == 0 && (!batch->token_ids_present || !batch->token_ids))
        return yvex_refuse(err, YVEX_ERR_BOUNDS, where, "MoE hash router requires token IDs");
    if (streams > 1ull) {
        const unsigned long long mix_rows = (streams + 2ull) * streams;
        coeff_count[0] = g.hidden; coeff_count[1] = mix_rows * streams * g.hidden; coeff_count[2] = mix_rows; coeff_count[3] = 3ull;
        for (int i = 0; i < 4; ++i) {
            /* F32 or BF16, like the reference's flat coefficient decoder (src/graph/moe.c:405-428) */
            const yvex_moe_weight_view *v = &job->weights[coeff[i]];
            if (!addr[coeff[i]]) return yvex_refuse(err, YVEX_ERR_STATE, where, "mHC envelope coefficients are not resident on this backend");
            if (!((v->qtype == 0u && v->encoded_bytes == coeff_count[i] * 4ull) || (v->qtype == 30u && v->encoded_bytes == coeff_count[i] * 2ull)))
                return yvex_refuse(err, YVEX_ERR_UNSUPPORTED, where, "mHC envelope coefficients must be F32 or BF16 tensors of the layer's geometry");
        }
        if (host_logits || tensor_logits)
            return yvex_refuse(err, YVEX_ERR_UNSUPPORTED, where, "supplied router logits cannot be combined with the mHC envelope");
        memset(&mhc, 0, sizeof(mhc));
        mhc.hidden = g.hidden; mhc.streams = streams; mhc.sinkhorn_iterations = layer->mhc_sinkhorn_iterations;
        mhc.rms_epsilon = layer->rms_epsilon; mhc.mhc_epsilon = layer->mhc_epsilon; mhc.post_multiplier = layer->mhc_post_multiplier;
        mhc.norm = (const float *)addr[YVEX_MOE_WEIGHT_FFN_NORM];
        mhc.mhc_fn = (const float *)addr[YVEX_MOE_WEIGHT_MHC_FUNCTION];
        mhc.base = (const float *)addr[YVEX_MOE_WEIGHT_MHC_BASE];
        mhc.scale = (const float *)addr[YVEX_MOE_WEIGHT_MHC_SCALE];
        mhc_ws = yvex_b200_mhc_workspace_bytes(streams, rows);
    }

    hid_bytes = rows * g.hidden * 4ull;
    in_bytes = hid_bytes * streams;
    kernel_ws = wide ? yvex_b200_moe_wide_workspace_bytes(&g, rows) : yvex_b200_moe_workspace_bytes(&g, rows);
    list_ws = yvex_b200_expert_worklist_workspace_bytes(rows * g.topk, g.experts);      /* reuses the kernel scratch afterwards */
    if (kernel_ws < list_ws) kernel_ws = list_ws;
    tensor_path = wide ? (unsigned long long)yvex_b200_moe_wide_uses_gemm(&g, &w) : 1ull;
    want_parts = output && (output->routed_rows || output->shared_rows);
    need = staging_bytes(&g, rows, streams) + kernel_ws;
    if (!backend->workspace || backend->workspace->bytes < need)
        return yvex_refuse(err, YVEX_ERR_NOMEM, where, "attached device workspace is smaller than workspace_required");
    ws_in = yvex_workspace_take(backend, &cursor, in_bytes);
    ws_out = yvex_workspace_take(backend, &cursor, in_bytes);
    ws_logits = yvex_workspace_take(backend, &cursor, rows * g.experts * 4ull);
    ws_sel = yvex_workspace_take(backend, &cursor, rows * g.topk * 4ull);
    ws_wts = yvex_workspace_take(backend, &cursor, rows * g.topk * 4ull);
    ws_ids = yvex_workspace_take(backend, &cursor, rows * 4ull);
    ws_kernel = yvex_workspace_take(backend, &cursor, kernel_ws);
    if (want_parts) {
        ws_routed = yvex_workspace_take(backend, &cursor, hid_bytes);
        ws_shared = yvex_workspace_take(backend, &cursor, hid_bytes);
        if (!ws_routed || !ws_shared) return yvex_refuse(err, YVEX_ERR_NOMEM, where, "attached device workspace is smaller than workspace_required");
    }
    if (streams > 1ull) {
        ws_norm = yvex_workspace_take(backend, &cursor, hid_bytes);
        ws_core = yvex_workspace_take(backend, &cursor, hid_bytes);
        ws_post = yvex_workspace_take(backend, &cursor, rows * streams * 4ull);
        ws_comb = yvex_workspace_take(backend, &cursor, rows * streams * streams * 4ull);
        ws_mhc = yvex_workspace_take(backend, &cursor, mhc_ws);
        for (int i = 0; i < 4; ++i) ws_coeff[i] = yvex_workspace_take(backend, &cursor, coeff_count[i] * 4ull);
    }
    if (!ws_in || !ws_out || !ws_logits || !ws_sel || !ws_wts || !ws_ids || !ws_kernel ||
        (streams > 1ull && (!ws_norm || !ws_core || !ws_post || !ws_comb || !ws_mhc || !ws_coeff[0] || !ws_coeff[1] || !ws_coeff[2] || !ws_coeff[3])))
        return yvex_refuse(err, YVEX_ERR_NOMEM, where, "attached device workspace is smaller than workspace_required");

    defer = job->device_completion && job->device_completion->defer && job->device_completion->host;
    /* the copy pipeline: host rows in, host rows out, no envelope, nothing deferred */
    pipelined = wide && batch->expanded_rows && !batch->device_outputs && output && output->combined_rows && !defer && streams == 1ull &&
                !tensor_logits && !want_parts;
    backend->last_pipeline_chunks = 0ull;
    if (pipelined) chunks = wide_chunks(&g, rows);
    if (chunks < 2ull) pipelined = 0;
    if (output && output->combined_rows && output->combined_capacity < rows * g.hidden * streams)
        return yvex_refuse(err, YVEX_ERR_BOUNDS, where, "combined output capacity is too small");
    sel_count = rows * g.topk;
    if (output && (output->selected_experts || output->selected_weights) && output->selection_capacity < sel_count)
        return yvex_refuse(err, YVEX_ERR_BOUNDS, where, "selection output capacity is too small");
    if (output && ((output->routed_rows && output->routed_capacity < rows * g.hidden) ||
                   (output->shared_rows && output->shared_capacity < rows * g.hidden) ||
                   (output->post_rows && output->post_capacity < rows * streams) ||
                   (output->combination_rows && output->combination_capacity < rows * streams * streams)))
        return yvex_refuse(err, YVEX_ERR_BOUNDS, where, "a partial output's capacity is too small");
    if (batch->device_rows) {
        if (!yvex_tensor_owned(backend, batch->device_rows) || !batch->device_rows->is_written ||
            batch->device_rows->dtype != YVEX_DTYPE_F32 || batch->device_rows->bytes < in_bytes)
            return yvex_refuse(err, YVEX_ERR_FORMAT, where, "device rows must be a written F32 tensor of this backend");
        dev_in = (const float *)batch->device_rows->data;
    } else {
        if (!pipelined && cudaMemcpyAsync(ws_in, batch->expanded_rows, in_bytes, cudaMemcpyHostToDevice, backend->stream) != cudaSuccess)
            return yvex_backend_fail(backend, where, err);
        result->h2d_bytes += in_bytes;
        result->upload_count++;
        dev_in = (const float *)ws_in;
    }
    if (tensor_logits) {
        if (!yvex_tensor_owned(backend, tensor_logits) || tensor_logits->bytes < rows * g.experts * 4ull)
            return yvex_refuse(err, YVEX_ERR_FORMAT, where, "device router logits must be an F32 tensor of this backend");
        dev_logits = (const float *)tensor_logits->data;
    } else if (host_logits) {
        if (!pipelined && cudaMemcpyAsync(ws_logits, host_logits, rows * g.experts * 4ull, cudaMemcpyHostToDevice, backend->stream) != cudaSuccess)
            return yvex_backend_fail(backend, where, err);
        result->h2d_bytes += rows * g.experts * 4ull;
        result->upload_count++;
        dev_logits = (const float *)ws_logits;
    }
    if (batch->token_ids_present && batch->token_ids) {
        if (!pipelined && cudaMemcpyAsync(ws_ids, batch->token_ids, rows * 4ull, cudaMemcpyHostToDevice, backend->stream) != cudaSuccess)
            return yvex_backend_fail(backend, where, err);
        result->h2d_bytes += rows * 4ull;
        result->upload_count++;
    }
    if (batch->device_outputs) {
        if (!yvex_tensor_owned(backend, batch->device_outputs) || batch->device_outputs->dtype != YVEX_DTYPE_F32 ||
            batch->device_outputs->bytes < in_bytes)
            return yvex_refuse(err, YVEX_ERR_FORMAT, where, "device outputs must be an F32 tensor of this backend");
        batch->device_outputs->is_written = 0;
        dev_out = (float *)batch->device_outputs->data;
    } else {
        if (!output || !output->combined_rows) return yvex_refuse(err, YVEX_ERR_INVALID_ARG, where, "a device or host output is required");
        dev_out = (float *)ws_out;
    }

    launches0 = yvex_b200_launch_count();
    memset(&run, 0, sizeof(run));
    run.backend = backend; run.job = job; run.g = g; run.w = w; run.mhc = mhc;
    run.streams = streams; run.rows = rows; run.mhc_ws = mhc_ws; run.kernel_ws = kernel_ws; run.tensor_path = tensor_path; run.wide = wide;
    run.provenance = (unsigned)batch->provenance <= 4u ? (unsigned)batch->provenance : rows == 1ull ? 0u : wide ? 3u : 2u;
    for (int i = 0; i < 4; ++i) {
        run.coeff_addr[i] = streams > 1ull ? addr[coeff[i]] : NULL;
        run.coeff_qtype[i] = streams > 1ull ? job->weights[coeff[i]].qtype : 0u;
        run.coeff_count[i] = coeff_count[i];
        run.ws_coeff[i] = ws_coeff[i];
    }
    run.dev_in = dev_in; run.dev_logits = dev_logits; run.dev_out = dev_out;
    run.ids = batch->token_ids_present && batch->token_ids ? (const uint32_t *)ws_ids : NULL;
    run.ws_norm = ws_norm; run.ws_core = ws_core; run.ws_post = ws_post; run.ws_comb = ws_comb; run.ws_mhc = ws_mhc;
    run.ws_routed = ws_routed; run.ws_shared = ws_shared; run.ws_sel = ws_sel; run.ws_wts = ws_wts; run.ws_kernel = ws_kernel;
    dev_obs = (yvex_expert_worklist_observation *)((unsigned char *)backend->status_word + YVEX_DEVICE_OBSERVATION_OFFSET);
    host_obs = (yvex_expert_worklist_observation *)(backend->host_scratch + YVEX_DEVICE_OBSERVATION_OFFSET);
    run.dev_obs = dev_obs;
    if (pipelined) {
        /* row range c: copied in on copy_in, computed on the backend's stream, copied out on copy_out */
        const unsigned char *host_in = (const unsigned char *)batch->expanded_rows, *host_lg = (const unsigned char *)host_logits;
        const int ids = batch->token_ids_present && batch->token_ids;
        int ok = cudaEventRecord(backend->ev_begin, backend->stream) == cudaSuccess &&
                 cudaStreamWaitEvent(backend->copy_in, backend->ev_begin, 0) == cudaSuccess &&
                 cudaStreamWaitEvent(backend->copy_out, backend->ev_begin, 0) == cudaSuccess;
        for (unsigned long long c = 0; c < chunks && ok; ++c) {
            const unsigned long long r0 = rows * c / chunks, n = rows * (c + 1ull) / chunks - r0;
            ok = cudaMemcpyAsync(ws_in + r0 * g.hidden * 4ull, host_in + r0 * g.hidden * 4ull, n * g.hidden * 4ull, cudaMemcpyHostToDevice,
                                 backend->copy_in) == cudaSuccess;
            if (ok && host_lg)
                ok = cudaMemcpyAsync(ws_logits + r0 * g.experts * 4ull, host_lg + r0 * g.experts * 4ull, n * g.experts * 4ull,
                                     cudaMemcpyHostToDevice, backend->copy_in) == cudaSuccess;
            if (ok && ids)
                ok = cudaMemcpyAsync(ws_ids + r0 * 4ull, batch->token_ids + r0, n * 4ull, cudaMemcpyHostToDevice, backend->copy_in) == cudaSuccess;
            ok = ok && cudaEventRecord(backend->ev_in[c], backend->copy_in) == cudaSuccess;
        }
        if (!ok) return yvex_backend_fail(backend, where, err);
        for (unsigned long long c = 0; c < chunks; ++c) {
            const unsigned long long r0 = rows * c / chunks, n = rows * (c + 1ull) / chunks - r0;
            if (cudaStreamWaitEvent(backend->stream, backend->ev_in[c], 0) != cudaSuccess) return yvex_backend_fail(backend, where, err);
            rc = yvex_b200_moe_wide(&g, &w, (const float *)ws_in + r0 * g.hidden, dev_logits ? dev_logits + r0 * g.experts : NULL,
                                    ids ? (const uint32_t *)ws_ids + r0 : NULL, n, (float *)ws_out + r0 * g.hidden,
                                    (int32_t *)ws_sel + r0 * g.topk, (float *)ws_wts + r0 * g.topk, ws_kernel, kernel_ws,
                                    backend->status_word, backend->stream);
            if (rc == YVEX_ERR_BACKEND) return yvex_backend_fail(backend, where, err);
            if (rc != YVEX_OK) return yvex_refuse(err, (yvex_status)rc, where, "device layer refused the MoE layer geometry");
            if (cudaEventRecord(backend->ev_done[c], backend->stream) != cudaSuccess ||
                cudaStreamWaitEvent(backend->copy_out, backend->ev_done[c], 0) != cudaSuccess ||
                cudaMemcpyAsync((unsigned char *)output->combined_rows + r0 * g.hidden * 4ull, ws_out + r0 * g.hidden * 4ull,
                                n * g.hidden * 4ull, cudaMemcpyDeviceToHost, backend->copy_out) != cudaSuccess)
                return yvex_backend_fail(backend, where, err);
        }
        /* the backend's stream ends behind the last copy out, so its synchronisation covers the whole call */
        if (cudaEventRecord(backend->ev_end, backend->copy_out) != cudaSuccess ||
            cudaStreamWaitEvent(backend->stream, backend->ev_end, 0) != cudaSuccess)
            return yvex_backend_fail(backend, where, err);
        result->d2h_bytes += in_bytes;
        result->download_count++;
        backend->last_pipeline_chunks = chunks;
        rc = rows_worklist(&run, &refusal);
    } else if (wide) {
        rc = rows_layer(&run, &refusal);
        if (rc == YVEX_OK) rc = rows_worklist(&run, &refusal);
    } else {
        /* the narrow entry replays a launch graph of this sequence once it has seen the combination (src/backend/cuda/moe.c:1645-1681) */
        rc = rows_enqueue_narrow(&run, want_parts, result, &graph_kernel_launches, &refusal);
    }
    if (rc == YVEX_ERR_BACKEND) return yvex_backend_fail(backend, where, err);
    if (rc != YVEX_OK) return yvex_refuse(err, (yvex_status)rc, where, refusal);
    if (!pipelined && output && output->combined_rows) {
        if (cudaMemcpyAsync(output->combined_rows, dev_out, in_bytes, cudaMemcpyDeviceToHost, backend->stream) != cudaSuccess)
            return yvex_backend_fail(backend, where, err);
        result->d2h_bytes += in_bytes;
        result->download_count++;
    }
    /* the parts of the sum and of the envelope, when the caller has room for them (src/runtime/moe.c:1501-1508) */
    {
        const struct { float *host; const unsigned char *dev; unsigned long long bytes; } part[4] = {
            {output ? output->routed_rows : NULL, ws_routed, hid_bytes},
            {output ? output->shared_rows : NULL, ws_shared, hid_bytes},
            {output && streams > 1ull ? output->post_rows : NULL, ws_post, rows * streams * 4ull},
            {output && streams > 1ull ? output->combination_rows : NULL, ws_comb, rows * streams * streams * 4ull}};
        for (int i = 0; i < 4; ++i) {
            if (!part[i].host || !part[i].dev) continue;
            if (cudaMemcpyAsync(part[i].host, part[i].dev, part[i].bytes, cudaMemcpyDeviceToHost, backend->stream) != cudaSuccess)
                return yvex_backend_fail(backend, where, err);
            result->d2h_bytes += part[i].bytes;
            result->download_count++;
        }
    }
    if (!defer && output && output->selected_weights) {
        if (cudaMemcpyAsync(output->selected_weights, ws_wts, sel_count * 4ull, cudaMemcpyDeviceToHost, backend->stream) != cudaSuccess)
            return yvex_backend_fail(backend, where, err);
        result->d2h_bytes += sel_count * 4ull;
        result->download_count++;
    }
    if (!defer && output && output->selected_experts) {
        /* int32 ids land in the upper half of the caller's u64 array and are widened in place after the sync */
        if (cudaMemcpyAsync((int32_t *)output->selected_experts + sel_count, ws_sel, sel_count * 4ull, cudaMemcpyDeviceToHost,
                            backend->stream) != cudaSuccess)
            return yvex_backend_fail(backend, where, err);
        result->d2h_bytes += sel_count * 4ull;
        result->download_count++;
    }
    /* into the backend's own page-locked scratch also when the completion is deferred: a copy into a slot in pageable
     * memory would hold the call until the stream has drained; complete_rows moves the summary and the status on */
    if (cudaMemcpyAsync(host_obs, dev_obs, sizeof(*dev_obs), cudaMemcpyDeviceToHost, backend->stream) != cudaSuccess)
        return yvex_backend_fail(backend, where, err);
    result->d2h_bytes += sizeof(*dev_obs);
    result->download_count++;
    /* counters as the reference publishes them (src/backend/cuda/moe.c:1757-1786) */
    result->row_count = rows;
    result->row_expert_pairs = sel_count;
    result->grouped_expert_operations = sel_count;
    result->shared_expert_operations = rows;
    result->expert_subviews_accessed = sel_count * 3ull;
    result->kernel_launches = graph_kernel_launches != ~0ull ? graph_kernel_launches : yvex_b200_launch_count() - launches0;
    /* launches whose contraction runs on the tensor cores: the gate/up and down kernels of each row range */
    result->tensor_core_launches = tensor_path ? 2ull * chunks : 0ull;
    if (streams > 1ull)
        result->active_weight_base_bytes += job->weights[YVEX_MOE_WEIGHT_FFN_NORM].encoded_bytes +
                                            job->weights[YVEX_MOE_WEIGHT_MHC_FUNCTION].encoded_bytes +
                                            job->weights[YVEX_MOE_WEIGHT_MHC_BASE].encoded_bytes +
                                            job->weights[YVEX_MOE_WEIGHT_MHC_SCALE].encoded_bytes;
    result->active_weight_base_bytes += job->weights[YVEX_MOE_WEIGHT_SHARED_GATE].encoded_bytes +
                                       job->weights[YVEX_MOE_WEIGHT_SHARED_UP].encoded_bytes +
                                       job->weights[YVEX_MOE_WEIGHT_SHARED_DOWN].encoded_bytes +
                                       job->weights[YVEX_MOE_WEIGHT_ROUTER].encoded_bytes;
    result->active_weight_per_unique_expert_bytes = (job->weights[YVEX_MOE_WEIGHT_ROUTED_GATE].encoded_bytes +
                                                     job->weights[YVEX_MOE_WEIGHT_ROUTED_UP].encoded_bytes +
                                                     job->weights[YVEX_MOE_WEIGHT_ROUTED_DOWN].encoded_bytes) / g.experts;
    result->schema_version = YVEX_MOE_ROW_BATCH_RESULT_SCHEMA_V4;
    result->execution_class = YVEX_EXECUTION_CLASS_DEVICE_NATIVE;
    result->memory.activation_bytes = 2ull * in_bytes;
    result->memory.temporary_bytes = need;
    result->memory.measured_operations = 1ull;
    if (defer) {
        yvex_moe_device_completion_slot *s = job->device_completion->host;
        s->status = 0;                       /* the worklist summary behind these fields is already on its way */
        s->pending = 1;
        s->row_count = rows;
        s->row_expert_pairs = sel_count;
        s->routed_experts = g.experts;
        s->active_base_bytes = result->active_weight_base_bytes;
        s->active_per_expert_bytes = result->active_weight_per_unique_expert_bytes;
        s->activation_bytes = result->memory.activation_bytes;
        s->temporary_bytes = result->memory.temporary_bytes;
        if (cudaMemcpyAsync(backend->host_scratch + YVEX_HOST_DEFERRED_STATUS_OFFSET, backend->status_word, sizeof(int), cudaMemcpyDeviceToHost,
                            backend->stream) != cudaSuccess)
            return yvex_backend_fail(backend, where, err);
        backend->pending_slot = s;
        result->device_completion_pending = 1;
        result->d2h_bytes += sizeof(int);
        if (batch->device_outputs) batch->device_outputs->is_written = 1;   /* stream-ordered for device consumers */
        yvex_error_clear(err);
        return YVEX_OK;
    }
    if (!yvex_backend_take_status(backend, &code)) return yvex_backend_fail(backend, where, err);
    result->stream_synchronizations = 1;
    result->d2h_bytes += sizeof(int);
    result->download_count++;
    if (code) { memset(result, 0, sizeof(*result)); return status_error(code, err); }
    if (!host_obs->bucket_count || host_obs->bucket_count > g.experts || !host_obs->maximum_bucket_population ||
        host_obs->narrow_pairs != sel_count - host_obs->tensor_core_eligible_pairs) {       /* src/backend/cuda/moe.c:1744-1755 */
        memset(result, 0, sizeof(*result));
        return yvex_refuse(err, YVEX_ERR_STATE, where, "CUDA expert worklist completion is invalid");
    }
    result->worklists = *host_obs;
    result->worklists.tensor_core_executed_pairs = result->worklists.tensor_core_eligible_pairs;
    result->unique_experts = host_obs->bucket_count;
    /* every active weight byte once: the replicated tensors plus the experts some row selected (:1905-1915) */
    result->memory.active_weight_bytes = result->active_weight_base_bytes + result->active_weight_per_unique_expert_bytes * result->unique_experts;
    result->memory.complete = 1;
    result->encoded_bytes_read = result->memory.active_weight_bytes;
    if (output && output->selected_experts) {
        const int32_t *src = (const int32_t *)output->selected_experts + sel_count;
        for (unsigned long long i = 0; i < sel_count; ++i) output->selected_experts[i] = (unsigned long long)src[i];
    }
    if (batch->device_outputs) batch->device_outputs->is_written = 1;
    result->completed = 1;
    yvex_error_clear(err);
    return YVEX_OK;
}

static int moe_execute_rows(yvex_backend *backend, const yvex_moe_layer_job *job, const yvex_moe_row_batch *batch,
                            const yvex_moe_row_batch_output *output, yvex_moe_row_batch_result *result, yvex_error *err) {
    return moe_execute(backend, job, batch, output, result, err, 0);
}

static int moe_execute_rows_wide(yvex_backend *backend, const yvex_moe_layer_job *job, const yvex_moe_row_batch *batch,
                                 const yvex_moe_row_batch_output *output, yvex_moe_row_batch_result *result, yvex_error *err) {
    return moe_execute(backend, job, batch, output, result, err, 1);
}

/* Deferred completion: one stream synchronisation, then the status slot decides (src/backend/cuda/moe.c:1925-1966). */
static int moe_complete_rows(yvex_backend *backend, int barrier_observed, yvex_moe_row_batch_result *result, yvex_error *err) {
    yvex_moe_device_completion_slot *s;
    int rc = yvex_backend_admit(backend, "cuda.moe.complete_rows", err), code;
    if (rc != YVEX_OK) return rc;
    s = backend->pending_slot;
    if (!s) return yvex_refuse(err, YVEX_ERR_STATE, "cuda.moe.complete_rows", "no deferred MoE completion is pending");
    if (!barrier_observed && cudaStreamSynchronize(backend->stream) != cudaSuccess)
        return yvex_backend_fail(backend, "cuda.moe.complete_rows", err);
    backend->pending_slot = NULL;
    s->pending = 0;
    s->worklist = *(const yvex_expert_worklist_observation *)(backend->host_scratch + YVEX_DEVICE_OBSERVATION_OFFSET);
    s->status = *(const int *)(backend->host_scratch + YVEX_HOST_DEFERRED_STATUS_OFFSET);
    code = s->status;
    if (code && cudaMemsetAsync(backend->status_word, 0, sizeof(int), backend->stream) != cudaSuccess)
        return yvex_backend_fail(backend, "cuda.moe.complete_rows", err);
    if (result) {
        result->device_completion_pending = 0;
        result->completed = code == 0;
        result->stream_synchronizations += barrier_observed ? 0ull : 1ull;
        if (!code) {
            result->worklists = s->worklist;
            result->worklists.tensor_core_executed_pairs = s->worklist.tensor_core_eligible_pairs;
            result->unique_experts = s->worklist.bucket_count;
            s->tensor_core_executed_pairs = s->worklist.tensor_core_eligible_pairs;
            result->memory.active_weight_bytes = result->active_weight_base_bytes + result->active_weight_per_unique_expert_bytes * result->unique_experts;
            result->memory.complete = 1;
            result->encoded_bytes_read = result->memory.active_weight_bytes;
        }
    }
    if (code) return status_error(code, err);
    yvex_error_clear(err);
    return YVEX_OK;
}

/* ---- token-local transaction (src/backend/cuda/moe.c:504-848) ---------------------------------------- */

static unsigned long long monotonic_ns(void) {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (unsigned long long)ts.tv_sec * 1000000000ull + (unsigned long long)ts.tv_nsec;
}

struct yvex_backend_moe_execution {
    yvex_backend *backend;
    const yvex_moe_layer_job *job;
    yvex_b200_moe_geometry g;
    yvex_b200_mhc mhc;
    unsigned long long streams, scratch_bytes;
    const float *expanded;                     /* device: the expanded input row */
    float *normalized, *post, *combination, *logits, *scores, *weights;
    int32_t *selected;
    float *gate, *up, *mid, *expert, *routed, *shared, *combined;
    unsigned long long launches0, h2d, d2h, uploads, downloads, subviews, direct_weights, syncs, d2d;
    unsigned long long started_ns, ingress_ns, routing_ns, routed_ns, shared_ns, sync_ns;
    int full_evidence, grouped_selected, finished;
};

#define TOKEN_FULL_EVIDENCE 3                  /* YVEX_ATTENTION_EVIDENCE_FULL */

static int token_device_rc(yvex_backend *backend, int rc, const char *where, const char *message, yvex_error *err) {
    if (rc == YVEX_OK) return YVEX_OK;
    if (rc == YVEX_ERR_BACKEND) return yvex_backend_fail(backend, where, err);
    return yvex_refuse(err, (yvex_status)rc, where, message);
}

static int token_download(yvex_backend_moe_execution *x, void *host, const void *dev, unsigned long long bytes, const char *where, yvex_error *err) {
    if (cudaMemcpyAsync(host, dev, bytes, cudaMemcpyDeviceToHost, x->backend->stream) != cudaSuccess)
        return yvex_backend_fail(x->backend, where, err);
    x->d2h += bytes;
    x->downloads++;
    return YVEX_OK;
}

static int token_sync(yvex_backend_moe_execution *x, const char *where, yvex_error *err) {
    const unsigned long long t0 = monotonic_ns();
    int code;
    if (!yvex_backend_take_status(x->backend, &code)) return yvex_backend_fail(x->backend, where, err);
    x->sync_ns += monotonic_ns() - t0;
    x->syncs++;
    x->d2h += sizeof(int);
    return status_error(code, err);
}

/* One expert: gate and up matvecs, SwiGLU * weight -> bf16, down matvec -> bf16, added to `aggregate`. */
static int token_expert(yvex_backend_moe_execution *x, const yvex_moe_weight_view *gate, const void *gate_at, const yvex_moe_weight_view *up,
                        const void *up_at, const yvex_moe_weight_view *down, const void *down_at, float weight, float *aggregate,
                        yvex_error *err) {
    yvex_backend *b = x->backend;
    const unsigned long long inter = gate->row_count, hidden = x->g.hidden;
    int rc = yvex_b200_gemv(gate->qtype, gate_at, inter, hidden, gate->row_bytes, x->normalized, 1ull, NULL, x->gate, 0, b->status_word, b->stream);
    if (rc == YVEX_OK)
        rc = yvex_b200_gemv(up->qtype, up_at, inter, hidden, up->row_bytes, x->normalized, 1ull, NULL, x->up, 0, b->status_word, b->stream);
    if (rc == YVEX_OK) rc = yvex_b200_moe_token_swiglu(x->gate, x->up, inter, x->g.limit, weight, x->mid, b->status_word, b->stream);
    if (rc == YVEX_OK)
        rc = yvex_b200_gemv(down->qtype, down_at, hidden, inter, down->row_bytes, x->mid, 1ull, NULL, x->expert, 1, b->status_word, b->stream);
    if (rc == YVEX_OK) rc = yvex_b200_moe_token_accumulate(x->expert, hidden, aggregate, b->status_word, b->stream);
    return token_device_rc(b, rc, "cuda.moe.add_expert", "device layer refused the expert geometry", err);
}

static int token_expert_views(yvex_backend_moe_execution *x, const yvex_moe_weight_view *gate, const yvex_moe_weight_view *up,
                              const yvex_moe_weight_view *down, float weight, int shared, yvex_error *err) {
    const char *where = "cuda.moe.add_expert";
    const yvex_moe_weight_view *v[3] = {gate, up, down};
    const void *at[3];
    const unsigned long long started = monotonic_ns();
    int rc;
    if (gate->row_count != up->row_count || down->row_width != gate->row_count || down->row_count != x->g.hidden ||
        gate->row_width != x->g.hidden || up->row_width != x->g.hidden)
        return yvex_refuse(err, YVEX_ERR_INVALID_ARG, where, "CUDA MoE expert geometry is invalid");
    if (gate->row_count > token_inter(&x->g)) return yvex_refuse(err, YVEX_ERR_BOUNDS, where, "expert is wider than the layer's intermediate width");
    for (int i = 0; i < 3; ++i) {
        if (!family_admitted(v[i]->kernel_family) || v[i]->layout == YVEX_EXECUTION_LAYOUT_DERIVED_BACKEND)
            return yvex_refuse(err, YVEX_ERR_UNSUPPORTED, where, "kernel family or weight layout is not one this backend executes");
        if (!yvex_b200_qtype_supported(v[i]->qtype))
            return yvex_refuse(err, YVEX_ERR_UNSUPPORTED, where, "expert qtype has no device decoder in this backend");
        if (!view_consistent(v[i], v[i]->row_count, v[i]->row_width))
            return yvex_refuse(err, YVEX_ERR_FORMAT, where, "expert weight view is inconsistent with its qtype");
        if (!resolve_view(x->backend, v[i], 1, &at[i]))
            return yvex_refuse(err, YVEX_ERR_STATE, where, "MoE weights are not resident on this backend");
    }
    rc = token_expert(x, gate, at[0], up, at[1], down, at[2], shared ? 1.0f : weight, shared ? x->shared : x->routed, err);
    if (rc != YVEX_OK) return rc;
    x->direct_weights += 3ull;
    x->subviews += shared ? 0ull : 3ull;
    if (shared) x->shared_ns += monotonic_ns() - started;
    else x->routed_ns += monotonic_ns() - started;
    return YVEX_OK;
}

/* The selected experts out of the routed packs, in rank order (moe_cuda_add_selected, src/backend/cuda/moe.c:586-671). */
static int token_add_selected(yvex_backend_moe_execution *x, const yvex_moe_router_result *router, yvex_error *err) {
    const yvex_moe_layer_job *job = x->job;
    static const int slots[3] = {YVEX_MOE_WEIGHT_ROUTED_GATE, YVEX_MOE_WEIGHT_ROUTED_UP, YVEX_MOE_WEIGHT_ROUTED_DOWN};
    const unsigned long long rows_per[3] = {x->g.inter, x->g.inter, x->g.hidden}, width[3] = {x->g.hidden, x->g.hidden, x->g.inter};
    for (int i = 0; i < 3; ++i)
        if (!view_consistent(&job->weights[slots[i]], x->g.experts * rows_per[i], width[i]))
            return yvex_refuse(err, YVEX_ERR_FORMAT, "cuda.moe.begin", "CUDA grouped selected-expert geometry is incompatible");
    for (unsigned long long rank = 0; rank < router->selected_count; ++rank) {
        yvex_moe_weight_view v[3];
        const unsigned long long e = router->selected_experts[rank];
        int rc;
        if (e >= x->g.experts) return yvex_refuse(err, YVEX_ERR_BOUNDS, "cuda.moe.begin", "router selected an expert outside the layer");
        for (int i = 0; i < 3; ++i) {
            const unsigned long long offset = e * rows_per[i] * job->weights[slots[i]].row_bytes;
            v[i] = job->weights[slots[i]];
            v[i].expert_index = e;
            v[i].row_count = rows_per[i];
            v[i].encoded_bytes = v[i].storage_bytes = (size_t)(rows_per[i] * v[i].row_bytes);
            v[i].encoded = v[i].encoded ? v[i].encoded + offset : NULL;
            v[i].device_address += offset;
        }
        rc = token_expert_views(x, &v[0], &v[1], &v[2], router->selected_weights[rank], 0, err);
        if (rc != YVEX_OK) return rc;
    }
    return YVEX_OK;
}

int yvex_backend_moe_close(yvex_backend_moe_execution **execution, yvex_error *err) {
    if (execution && *execution) {
        free(*execution);
        *execution = NULL;
    }
    yvex_error_clear(err);
    return YVEX_OK;
}

int yvex_backend_moe_begin(yvex_backend_moe_execution **out, yvex_backend *backend, const yvex_moe_layer_job *job,
                           yvex_moe_layer_result *result, yvex_error *err) {
    const char *where = "cuda.moe.begin";
    const yvex_moe_layer_plan *layer = job ? job->layer : NULL;
    static const int coeff[4] = {YVEX_MOE_WEIGHT_FFN_NORM, YVEX_MOE_WEIGHT_MHC_FUNCTION, YVEX_MOE_WEIGHT_MHC_BASE, YVEX_MOE_WEIGHT_MHC_SCALE};
    static const int routing[3] = {YVEX_MOE_WEIGHT_ROUTER, YVEX_MOE_WEIGHT_ROUTER_TABLE, YVEX_MOE_WEIGHT_ROUTER_BIAS};
    yvex_backend_moe_execution *x;
    yvex_b200_moe_weights w;
    unsigned long long cursor = 0, streams, in_bytes, hid_bytes, inter_bytes, coeff_count[4] = {0, 0, 0, 0}, mhc_ws = 0, routed_started;
    unsigned char *ws_in, *ws_token, *ws_mhc = NULL, *ws_coeff[4] = {NULL, NULL, NULL, NULL};
    const void *addr[YVEX_MOE_WEIGHT_COUNT];
    const yvex_moe_weight_view *router;
    int rc;
    if (out) *out = NULL;
    if (!out || !backend || !job || !layer || !result || (!job->expanded_input && !job->device_input) || !result->combined_output ||
        result->combined_capacity < layer->hidden_width)
        return yvex_refuse(err, YVEX_ERR_INVALID_ARG, where, "CUDA MoE begin arguments are invalid");
    streams = envelope_streams(layer);
    if (streams > 1ull && (!result->post || result->post_capacity < streams || !result->combination || result->combination_capacity < streams * streams))
        return yvex_refuse(err, YVEX_ERR_INVALID_ARG, where, "CUDA MoE begin arguments are invalid");
    rc = yvex_backend_admit(backend, where, err);
    if (rc != YVEX_OK) return rc;
    if (backend->pending_slot) return yvex_refuse(err, YVEX_ERR_STATE, where, "a deferred MoE completion is still pending");
    if (yvex_test_seam("YVEX_TEST_CUDA_LAUNCH_FAILURE", "moe-token")) return yvex_backend_fail(backend, where, err);
    if (layer->expanded_width && layer->expanded_width != streams * layer->hidden_width)
        return yvex_refuse(err, YVEX_ERR_FORMAT, where, "expanded width is not residual streams x hidden width");
    if (streams > 1ull && layer->mhc_mixing_rows != (streams + 2ull) * streams)
        return yvex_refuse(err, YVEX_ERR_FORMAT, where, "mHC mixing rows must be (streams + 2) x streams");
    in_bytes = streams * layer->hidden_width * 4ull;
    if ((job->device_input || job->device_output) &&
        (!yvex_tensor_owned(backend, job->device_input) || !yvex_tensor_owned(backend, job->device_output) ||
         job->device_input->dtype != YVEX_DTYPE_F32 || job->device_output->dtype != YVEX_DTYPE_F32 || job->device_input->bytes != in_bytes ||
         job->device_output->bytes != in_bytes || !job->device_input->is_written))
        return yvex_refuse(err, YVEX_ERR_FORMAT, where, "CUDA MoE device activation views are incompatible");
    if (job->cancel_requested && job->cancel_requested(job->cancel_context))
        return yvex_refuse(err, YVEX_ERR_CANCELLED, where, "MoE execution was cancelled");
    x = (yvex_backend_moe_execution *)calloc(1u, sizeof(*x));
    if (!x) return yvex_refuse(err, YVEX_ERR_NOMEM, where, "CUDA MoE owner allocation failed");
    x->backend = backend;
    x->job = job;
    x->streams = streams;
    x->started_ns = monotonic_ns();
    x->launches0 = yvex_b200_launch_count();
    x->full_evidence = job->evidence_level == TOKEN_FULL_EVIDENCE;
    x->grouped_selected = job->device_output && !x->full_evidence && job->weights[YVEX_MOE_WEIGHT_ROUTED_GATE].device_address &&
                          job->weights[YVEX_MOE_WEIGHT_ROUTED_UP].device_address && job->weights[YVEX_MOE_WEIGHT_ROUTED_DOWN].device_address;
    plan_geometry(layer, job, &x->g);
#define TOKEN_FAIL(code_, message_) do { rc = yvex_refuse(err, (code_), where, (message_)); goto fail; } while (0)
    if (x->g.experts > 256ull || x->g.topk > YVEX_MOE_MAX_SELECTED || !x->g.topk || x->g.topk > x->g.experts)
        TOKEN_FAIL(YVEX_ERR_BOUNDS, "router geometry exceeds the router result's capacity");
    for (int i = 0; i < 3; ++i)
        if (!resolve_view(backend, &job->weights[routing[i]], 0, &addr[routing[i]])) TOKEN_FAIL(YVEX_ERR_STATE, "MoE weights are not resident on this backend");
    router = &job->weights[YVEX_MOE_WEIGHT_ROUTER];
    if (!addr[YVEX_MOE_WEIGHT_ROUTER]) TOKEN_FAIL(YVEX_ERR_STATE, "router weights are not resident on this backend");
    if (!yvex_b200_qtype_supported(router->qtype)) TOKEN_FAIL(YVEX_ERR_UNSUPPORTED, "router qtype has no device decoder in this backend");
    if (!view_consistent(router, x->g.experts, x->g.hidden)) TOKEN_FAIL(YVEX_ERR_FORMAT, "router weight view is inconsistent with the layer geometry");
    if (x->g.router_class == 0 && (!job->token_id_present || job->token_id >= layer->hash_table_rows || !addr[YVEX_MOE_WEIGHT_ROUTER_TABLE]))
        TOKEN_FAIL(YVEX_ERR_BOUNDS, "CUDA hash router token ID is invalid");
    memset(&w, 0, sizeof(w));
    w.router = router->qtype == 0u ? (const float *)addr[YVEX_MOE_WEIGHT_ROUTER] : NULL;
    w.bias = (const float *)addr[YVEX_MOE_WEIGHT_ROUTER_BIAS];
    w.hash_table = (const int32_t *)addr[YVEX_MOE_WEIGHT_ROUTER_TABLE];
    if (streams > 1ull) {
        const unsigned long long mix_rows = (streams + 2ull) * streams;
        coeff_count[0] = x->g.hidden; coeff_count[1] = mix_rows * streams * x->g.hidden; coeff_count[2] = mix_rows; coeff_count[3] = 3ull;
        for (int i = 0; i < 4; ++i) {
            const yvex_moe_weight_view *v = &job->weights[coeff[i]];
            if (!resolve_view(backend, v, 1, &addr[coeff[i]])) TOKEN_FAIL(YVEX_ERR_STATE, "mHC envelope coefficients are not resident on this backend");
            if (!((v->qtype == 0u && v->encoded_bytes == coeff_count[i] * 4ull) || (v->qtype == 30u && v->encoded_bytes == coeff_count[i] * 2ull)))
                TOKEN_FAIL(YVEX_ERR_UNSUPPORTED, "mHC envelope coefficients must be F32 or BF16 tensors of the layer's geometry");
        }
        x->mhc.hidden = x->g.hidden; x->mhc.streams = streams; x->mhc.sinkhorn_iterations = layer->mhc_sinkhorn_iterations;
        x->mhc.rms_epsilon = layer->rms_epsilon; x->mhc.mhc_epsilon = layer->mhc_epsilon; x->mhc.post_multiplier = layer->mhc_post_multiplier;
        x->mhc.norm = (const float *)addr[YVEX_MOE_WEIGHT_FFN_NORM];
        x->mhc.mhc_fn = (const float *)addr[YVEX_MOE_WEIGHT_MHC_FUNCTION];
        x->mhc.base = (const float *)addr[YVEX_MOE_WEIGHT_MHC_BASE];
        x->mhc.scale = (const float *)addr[YVEX_MOE_WEIGHT_MHC_SCALE];
        mhc_ws = yvex_b200_mhc_workspace_bytes(streams, 1ull);
    }
    /* ranges of the attached workspace, from its start: a transaction owns it until finish */
    hid_bytes = x->g.hidden * 4ull;
    inter_bytes = token_inter(&x->g) * 4ull;
    ws_in = yvex_workspace_take(backend, &cursor, in_bytes);
    x->normalized = (float *)yvex_workspace_take(backend, &cursor, hid_bytes);
    x->expert = (float *)yvex_workspace_take(backend, &cursor, hid_bytes);
    x->routed = (float *)yvex_workspace_take(backend, &cursor, hid_bytes);
    x->shared = (float *)yvex_workspace_take(backend, &cursor, hid_bytes);
    x->combined = (float *)yvex_workspace_take(backend, &cursor, hid_bytes);
    x->gate = (float *)yvex_workspace_take(backend, &cursor, inter_bytes);
    x->up = (float *)yvex_workspace_take(backend, &cursor, inter_bytes);
    x->mid = (float *)yvex_workspace_take(backend, &cursor, inter_bytes);
    x->logits = (float *)yvex_workspace_take(backend, &cursor, x->g.experts * 4ull);
    x->scores = (float *)yvex_workspace_take(backend, &cursor, x->g.experts * 4ull);
    x->selected = (int32_t *)yvex_workspace_take(backend, &cursor, x->g.topk * 4ull);
    x->weights = (float *)yvex_workspace_take(backend, &cursor, x->g.topk * 4ull);
    ws_token = yvex_workspace_take(backend, &cursor, 4ull);
    if (streams > 1ull) {
        x->post = (float *)yvex_workspace_take(backend, &cursor, streams * 4ull);
        x->combination = (float *)yvex_workspace_take(backend, &cursor, streams * streams * 4ull);
        ws_mhc = yvex_workspace_take(backend, &cursor, mhc_ws);
        for (int i = 0; i < 4; ++i) ws_coeff[i] = yvex_workspace_take(backend, &cursor, coeff_count[i] * 4ull);
    }
    if (!ws_in || !x->normalized || !x->expert || !x->routed || !x->shared || !x->combined || !x->gate || !x->up || !x->mid || !x->logits ||
        !x->scores || !x->selected || !x->weights || !ws_token ||
        (streams > 1ull && (!x->post || !x->combination || !ws_mhc || !ws_coeff[0] || !ws_coeff[1] || !ws_coeff[2] || !ws_coeff[3])))
        TOKEN_FAIL(YVEX_ERR_NOMEM, "attached device workspace is smaller than workspace_required");
    x->scratch_bytes = cursor;
#define TOKEN_CUDA(call_) do { if ((call_) != cudaSuccess) { rc = yvex_backend_fail(backend, where, err); goto fail; } } while (0)
#define TOKEN_DEVICE(call_, message_) do { rc = token_device_rc(backend, (call_), where, (message_), err); if (rc != YVEX_OK) goto fail; } while (0)
    /* ingress */
    if (job->device_input) {
        x->expanded = (const float *)job->device_input->data;
    } else {
        TOKEN_CUDA(cudaMemcpyAsync(ws_in, job->expanded_input, in_bytes, cudaMemcpyHostToDevice, backend->stream));
        x->h2d += in_bytes;
        x->uploads++;
        x->expanded = (const float *)ws_in;
    }
    TOKEN_CUDA(cudaMemsetAsync(x->routed, 0, hid_bytes, backend->stream));
    TOKEN_CUDA(cudaMemsetAsync(x->shared, 0, hid_bytes, backend->stream));
    if (streams > 1ull) {
        const float **slot_ptr[4] = {&x->mhc.norm, &x->mhc.mhc_fn, &x->mhc.base, &x->mhc.scale};
        for (int i = 0; i < 4; ++i) {
            if (job->weights[coeff[i]].qtype != 30u) continue;
            TOKEN_DEVICE(yvex_b200_dequant_rows(30u, addr[coeff[i]], 1ull, coeff_count[i], coeff_count[i] * 2ull, (float *)ws_coeff[i],
                                                backend->status_word, backend->stream), "device layer refused an mHC coefficient tensor");
            *slot_ptr[i] = (const float *)ws_coeff[i];
        }
        TOKEN_DEVICE(yvex_b200_mhc_prepare(&x->mhc, x->expanded, 1ull, x->normalized, x->post, x->combination, ws_mhc, mhc_ws,
                                           backend->status_word, backend->stream), "device layer refused the mHC envelope geometry");
    } else {
        TOKEN_DEVICE(yvex_b200_moe_token_round(x->expanded, x->g.hidden, x->normalized, backend->status_word, backend->stream),
                     "device layer refused the ingress row");
    }
    routed_started = monotonic_ns();
    x->ingress_ns = routed_started - x->started_ns;
    /* router: projection (double accumulation for F32 rows, the dequant matvec otherwise), scores, top-k or the hash row */
    if (x->g.router_class == 0) {
        TOKEN_CUDA(cudaMemcpyAsync(ws_token, &job->token_id, 4ull, cudaMemcpyHostToDevice, backend->stream));
        x->h2d += 4ull;
    }
    if (!w.router)
        TOKEN_DEVICE(yvex_b200_gemv(router->qtype, addr[YVEX_MOE_WEIGHT_ROUTER], x->g.experts, x->g.hidden, router->row_bytes, x->normalized, 1ull,
                                    NULL, x->logits, 0, backend->status_word, backend->stream), "device layer refused the router projection");
    TOKEN_DEVICE(yvex_b200_moe_route(&x->g, &w, x->normalized, w.router ? NULL : x->logits, x->g.router_class == 0 ? (const uint32_t *)ws_token : NULL,
                                     1ull, x->selected, x->weights, x->logits, NULL, 0ull, backend->status_word, backend->stream),
                 "device layer refused the router geometry");
    TOKEN_DEVICE(yvex_b200_moe_token_scores(x->logits, x->g.experts, x->scores, backend->status_word, backend->stream),
                 "device layer refused the router scores");
    x->direct_weights += 1ull + (w.bias ? 1ull : 0ull);
    {
        int32_t *host_selected = (int32_t *)(backend->host_scratch + 2048);
        memset(&result->router, 0, sizeof(result->router));
        if (!job->device_output || x->full_evidence) {
            rc = token_download(x, result->router.router_logits, x->logits, x->g.experts * 4ull, where, err);
            if (rc == YVEX_OK) rc = token_download(x, result->router.router_scores, x->scores, x->g.experts * 4ull, where, err);
            if (rc != YVEX_OK) goto fail;
        }
        rc = token_download(x, host_selected, x->selected, x->g.topk * 4ull, where, err);
        if (rc == YVEX_OK) rc = token_download(x, result->router.selected_weights, x->weights, x->g.topk * 4ull, where, err);
        if (rc == YVEX_OK) rc = token_sync(x, where, err);
        if (rc != YVEX_OK) goto fail;
        result->router.selected_count = x->g.topk;
        for (unsigned long long r = 0; r < x->g.topk; ++r)
            result->router.selected_experts[r] = host_selected[r] < 0 ? ~0ull : (unsigned long long)host_selected[r];
    }
    x->routing_ns = monotonic_ns() - routed_started;
    if (x->grouped_selected) {
        rc = token_add_selected(x, &result->router, err);
        if (rc != YVEX_OK) goto fail;
    }
    *out = x;
    yvex_error_clear(err);
    return YVEX_OK;
fail:
    free(x);
    return rc;
}

int yvex_backend_moe_add_expert(yvex_backend_moe_execution *execution, const yvex_moe_weight_view *gate, const yvex_moe_weight_view *up,
                                const yvex_moe_weight_view *down, float route_weight, int shared, yvex_error *err) {
    int rc;
    if (!execution || !execution->job || !gate || !up || !down || execution->finished)
        return yvex_refuse(err, YVEX_ERR_INVALID_ARG, "cuda.moe.add_expert", "CUDA MoE expert geometry is invalid");
    rc = yvex_backend_admit(execution->backend, "cuda.moe.add_expert", err);
    if (rc != YVEX_OK) return rc;
    rc = token_expert_views(execution, gate, up, down, route_weight, shared, err);
    if (rc == YVEX_OK) yvex_error_clear(err);
    return rc;
}

int yvex_backend_moe_finish(yvex_backend_moe_execution *execution, yvex_moe_layer_result *result, yvex_error *err) {
    const char *where = "cuda.moe.finish";
    yvex_backend_moe_execution *x = execution;
    const yvex_moe_layer_job *job = x ? x->job : NULL;
    yvex_backend *backend = x ? x->backend : NULL;
    unsigned long long hid_bytes;
    int rc;
    if (!x || !job || !result || x->finished) return yvex_refuse(err, YVEX_ERR_INVALID_ARG, where, "CUDA MoE finish is invalid");
    if (!result->routed_output || result->routed_capacity < x->g.hidden || !result->shared_output || result->shared_capacity < x->g.hidden)
        return yvex_refuse(err, YVEX_ERR_INVALID_ARG, where, "CUDA MoE routed/shared publication capacity is invalid");
    rc = yvex_backend_admit(backend, where, err);
    if (rc != YVEX_OK) return rc;
    hid_bytes = x->g.hidden * 4ull;
    rc = token_device_rc(backend, yvex_b200_moe_token_sum_round(x->routed, x->shared, x->g.hidden, x->combined, backend->status_word, backend->stream),
                         where, "device layer refused the combination", err);
    if (rc != YVEX_OK) return rc;
    if (job->device_output) {
        job->device_output->is_written = 0;
        if (x->streams > 1ull) {
            rc = token_device_rc(backend, yvex_b200_mhc_post(&x->mhc, x->combined, x->expanded, x->post, x->combination, 1ull,
                                                             (float *)job->device_output->data, backend->status_word, backend->stream),
                                 where, "device layer refused the mHC envelope geometry", err);
            if (rc != YVEX_OK) return rc;
        } else {
            if (cudaMemcpyAsync(job->device_output->data, x->combined, hid_bytes, cudaMemcpyDeviceToDevice, backend->stream) != cudaSuccess)
                return yvex_backend_fail(backend, where, err);
            x->d2d += hid_bytes;
        }
    }
    if (!job->device_output || x->full_evidence) {
        rc = token_download(x, result->combined_output, x->combined, hid_bytes, where, err);
        if (rc == YVEX_OK) rc = token_download(x, result->routed_output, x->routed, hid_bytes, where, err);
        if (rc == YVEX_OK) rc = token_download(x, result->shared_output, x->shared, hid_bytes, where, err);
        if (rc == YVEX_OK && x->streams > 1ull) rc = token_download(x, result->post, x->post, x->streams * 4ull, where, err);
        if (rc == YVEX_OK && x->streams > 1ull)
            rc = token_download(x, result->combination, x->combination, x->streams * x->streams * 4ull, where, err);
        if (rc != YVEX_OK) return rc;
    }
    rc = token_sync(x, where, err);
    if (rc != YVEX_OK) return rc;
    if (job->device_output) job->device_output->is_written = 1;
    if (job->device_input && job->device_output) {
        result->memory.activation_bytes = 2ull * x->streams * hid_bytes;
        result->memory.temporary_bytes = x->scratch_bytes;
    }
    result->expert_subviews_accessed += x->subviews;
    result->host_to_device_bytes += x->h2d;
    result->device_to_host_bytes += x->d2h;
    result->kernel_launches += yvex_b200_launch_count() - x->launches0;
    result->upload_count += x->uploads;
    result->download_count += x->downloads;
    result->cache_hits += x->direct_weights;
    result->device_to_device_bytes += x->d2d;
    result->stream_synchronizations += x->syncs;
    result->synchronization_ns += x->sync_ns;
    result->ingress_ns += x->ingress_ns;
    result->routing_ns += x->routing_ns;
    result->routed_ns += x->routed_ns;
    result->shared_ns += x->shared_ns;
    result->total_ns += monotonic_ns() - x->started_ns;
    x->finished = 1;
    yvex_error_clear(err);
    return YVEX_OK;
}

static const yvex_backend_moe_operations moe_operations = {
    derived_plan, derived_build, moe_workspace_required, moe_execute_rows, moe_complete_rows,
    moe_workspace_required_wide, moe_execute_rows_wide};

unsigned long long yvex_backend_moe_last_pipeline_chunks(const yvex_backend *backend) {
    return backend ? backend->last_pipeline_chunks : 0ull;
}

const yvex_backend_moe_operations *yvex_backend_moe_operations_get(const yvex_backend *backend) {
    if (!backend || backend->kind != YVEX_BACKEND_KIND_CUDA || backend->closing ||
        atomic_load(&((yvex_backend *)backend)->status) == YVEX_BACKEND_STATUS_FAILED)
        return NULL;
    return &moe_operations;
}

/* ---- helpers shared with the expert-parallel entry (host/ep.c) ------------------------------------------ */
int yvex_moe_plan_geometry(const yvex_moe_layer_plan *layer, const yvex_moe_layer_job *job, yvex_b200_moe_geometry *g) { return plan_geometry(layer, job, g); }
int yvex_moe_resolve_view(const yvex_backend *backend, const yvex_moe_weight_view *v, int required, const void **out) { return resolve_view(backend, v, required, out); }
int yvex_moe_view_consistent(const yvex_moe_weight_view *v, unsigned long long rows, unsigned long long width) { return view_consistent(v, rows, width); }
int yvex_moe_status_error(int code, yvex_error *err) { return status_error(code, err); }
