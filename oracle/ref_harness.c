/*
 * TEST INFRASTRUCTURE - not part of the shipped library.
 *
 * Thin plain-pointer entry points over the UNMODIFIED reference library (compiled from its own
 * sources by oracle/Makefile into oracle/_ref/libyvex_ref.so). Every numeric result below is
 * produced by a reference function; this file only builds the argument structs those functions
 * take and fans independent tokens/rows out over threads. Loaded with ctypes by the tests, by
 * the fixture generator and by bench.py's CPU-baseline legs; never by the product path.
 *
 * Reference entry points used:
 *   yvex_gguf_qtype_geometry_find      src/gguf/qtype.c
 *   yvex_quant_numeric_capability_at   src/gguf/quant_registry.c:113
 *   yvex_quant_decode_block            src/gguf/quant_block.c:769
 *   yvex_quant_cpu_dot                 src/gguf/quant_compute.c:116
 *   yvex_quant_{f16,bf16}_{decode,encode}  src/gguf/quant_scalar.c:40-143
 *   yvex_moe_route_cpu                 src/graph/moe.c:520
 *   yvex_moe_expert_cpu                src/graph/moe.c:587
 *   yvex_backend_op_attention (CPU)    src/backend/core.c:990, src/backend/cpu.c:319
 *   yvex_moe_input_seal / _write       src/runtime/moe_input.c:196, :279 (fixture files for the reader tests)
 * The routed+shared combine restates the ten lines of src/runtime/moe.c:607-632 because that
 * function is static and needs a full runtime context.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <yvex/backend.h>
#include <yvex/core.h>
#include <yvex/qtype.h>
#include <yvex/internal/backend.h>
#include <yvex/internal/moe.h>
#include <yvex/internal/quant_numeric.h>
#include "src/graph/private.h"      /* yvex_attention_mhc_post and its argument struct */

#define REF_MAX_THREADS 256

int ref_qtype_geometry(unsigned int qtype, unsigned long long *block_elements,
                       unsigned long long *block_bytes) {
    const yvex_gguf_qtype_geometry *g = yvex_gguf_qtype_geometry_find(qtype);
    if (!g) return YVEX_ERR_UNSUPPORTED;
    *block_elements = g->block_size;
    *block_bytes = g->bytes_per_block;
    return YVEX_OK;
}

/* flags: bit0 storage, bit1 encoder, bit2 decoder, bit3 cpu compute, bit4 cuda compute. */
int ref_qtype_capability(unsigned int qtype) {
    const yvex_quant_numeric_capability *c = yvex_quant_numeric_capability_at(qtype);
    if (!c) return -1;
    return (c->storage_admitted ? 1 : 0) | (c->encoder_available ? 2 : 0) |
           (c->reference_decoder_available ? 4 : 0) |
           (c->dedicated_cpu_compute_available ? 8 : 0) |
           (c->dedicated_cuda_compute_available ? 16 : 0);
}

float ref_f16_decode(unsigned short bits) { return yvex_quant_f16_decode(bits); }
unsigned short ref_f16_encode(float v) { return yvex_quant_f16_encode(v); }
float ref_bf16_decode(unsigned short bits) { return yvex_quant_bf16_decode(bits); }
unsigned short ref_bf16_encode(float v) { return yvex_quant_bf16_encode(v); }

int ref_decode_block(unsigned int qtype, const unsigned char *encoded, size_t bytes, float *out,
                     unsigned long long elements) {
    yvex_error err;
    yvex_quant_failure failure;
    memset(&err, 0, sizeof(err));
    return yvex_quant_decode_block(qtype, encoded, bytes, out, elements, &failure, &err);
}

int ref_decode_rows(unsigned int qtype, const unsigned char *encoded, unsigned long long rows,
                    unsigned long long width, float *out) {
    const yvex_gguf_qtype_geometry *g = yvex_gguf_qtype_geometry_find(qtype);
    unsigned long long blocks, b;
    if (!g || !g->block_size || width % g->block_size) return YVEX_ERR_BOUNDS;
    blocks = rows * (width / g->block_size);
    for (b = 0; b < blocks; ++b) {
        int rc = ref_decode_block(qtype, encoded + b * g->bytes_per_block, g->bytes_per_block,
                                  out + b * g->block_size, g->block_size);
        if (rc != YVEX_OK) return rc;
    }
    return YVEX_OK;
}

typedef struct {
    unsigned int qtype;
    const unsigned char *encoded;
    unsigned long long row_begin, row_end, width, row_bytes;
    const float *x;
    float *y;
    int rc;
} ref_matvec_span;

static void *ref_matvec_worker(void *arg) {
    ref_matvec_span *s = (ref_matvec_span *)arg;
    unsigned long long r;
    for (r = s->row_begin; r < s->row_end; ++r) {
        yvex_error err;
        yvex_quant_failure failure;
        int rc;
        memset(&err, 0, sizeof(err));
        rc = yvex_quant_cpu_dot(s->qtype, s->encoded + r * s->row_bytes, (size_t)s->row_bytes,
                                s->x, s->width, &s->y[r], &failure, &err);
        if (rc != YVEX_OK) {
            s->rc = rc;
            return NULL;
        }
    }
    return NULL;
}

/* y[r] = yvex_quant_cpu_dot(row r, x); rows split over `threads` pthreads (1 = as written). */
int ref_matvec(unsigned int qtype, const unsigned char *encoded, unsigned long long rows,
               unsigned long long width, const float *x, float *y, int threads) {
    const yvex_gguf_qtype_geometry *g = yvex_gguf_qtype_geometry_find(qtype);
    ref_matvec_span spans[REF_MAX_THREADS];
    pthread_t tids[REF_MAX_THREADS];
    unsigned long long row_bytes;
    int t, rc = YVEX_OK;
    if (!g || !g->block_size || width % g->block_size) return YVEX_ERR_BOUNDS;
    row_bytes = width / g->block_size * g->bytes_per_block;
    if (threads < 1) threads = 1;
    if (threads > REF_MAX_THREADS) threads = REF_MAX_THREADS;
    for (t = 0; t < threads; ++t) {
        spans[t] = (ref_matvec_span){qtype, encoded, rows * t / threads, rows * (t + 1) / threads,
                                     width, row_bytes, x, y, YVEX_OK};
        if (threads == 1) ref_matvec_worker(&spans[t]);
        else if (pthread_create(&tids[t], NULL, ref_matvec_worker, &spans[t])) return YVEX_ERR;
    }
    for (t = 0; t < threads; ++t) {
        if (threads > 1) pthread_join(tids[t], NULL);
        if (spans[t].rc != YVEX_OK) rc = spans[t].rc;
    }
    return rc;
}

/* Plain description of one MoE layer; mirrors the fields of yvex_moe_layer_plan that the CPU
 * numerics read, plus the packed weight tensors (expert-major, canonical row layout). */
typedef struct {
    unsigned long long hidden, experts, topk, inter, shared_inter;
    double scaling, limit;
    int normalize, router_class; /* 1 learned, 0 hash */
    unsigned int gate_qtype, up_qtype, down_qtype;
    const float *router;          /* [experts x hidden] f32, or NULL when logits are given */
    const float *bias;            /* [experts] f32 or NULL (zero) */
    const int32_t *hash_table;    /* [hash_stored_rows x topk] */
    unsigned long long hash_rows, hash_stored_rows;
    const unsigned char *gate, *up, *down;                /* routed packs */
    const unsigned char *shared_gate, *shared_up, *shared_down;
} ref_moe_layer;

static unsigned long long ref_row_bytes(unsigned int qtype, unsigned long long width) {
    const yvex_gguf_qtype_geometry *g = yvex_gguf_qtype_geometry_find(qtype);
    return g && g->block_size ? width / g->block_size * g->bytes_per_block : 0;
}

static yvex_moe_weight_view ref_view(unsigned int qtype, const unsigned char *base,
                                     unsigned long long rows, unsigned long long width) {
    yvex_moe_weight_view v;
    memset(&v, 0, sizeof(v));
    v.qtype = qtype;
    v.encoded = base;
    v.row_width = width;
    v.row_count = rows;
    v.row_bytes = ref_row_bytes(qtype, width);
    v.encoded_bytes = v.storage_bytes = (size_t)(v.row_bytes * rows);
    return v;
}

static void ref_plan(const ref_moe_layer *L, yvex_moe_layer_plan *plan) {
    memset(plan, 0, sizeof(*plan));
    plan->schema_version = YVEX_MOE_PLAN_SCHEMA_V1;
    plan->router_class = L->router_class ? YVEX_MOE_ROUTER_LEARNED_HIDDEN_STATE
                                         : YVEX_MOE_ROUTER_HASH_TOKEN_ID;
    plan->hidden_width = L->hidden;
    plan->routed_experts = L->experts;
    plan->shared_experts = 1;
    plan->experts_per_token = L->topk;
    plan->expert_intermediate_width = L->inter;
    plan->shared_intermediate_width = L->shared_inter;
    plan->hash_table_rows = L->hash_rows;
    plan->routed_scaling_factor = L->scaling;
    plan->activation_limit = L->limit;
    plan->normalize_topk_probabilities = L->normalize;
}

/*
 * Route one token with yvex_moe_route_cpu. When L->router is NULL, `x_or_logits` holds the
 * router logits themselves: they are fed through an identity F32 router (exact: each dot has
 * one non-zero term), which is how the prefill configs supply logits directly.
 */
int ref_route(const ref_moe_layer *L, const float *x_or_logits, unsigned int token_id,
              int token_present, unsigned long long *selected, float *weights, float *logits,
              float *scores) {
    yvex_moe_layer_plan plan;
    yvex_moe_layer_job job;
    yvex_moe_router_result result;
    yvex_error err;
    float *identity = NULL, zero_bias[256];
    unsigned long long e, width = L->router ? L->hidden : L->experts;
    int rc;
    memset(&err, 0, sizeof(err));
    memset(&job, 0, sizeof(job));
    memset(zero_bias, 0, sizeof(zero_bias));
    ref_plan(L, &plan);
    job.layer = &plan;
    job.token_id = token_id;
    job.token_id_present = token_present;
    if (L->router) {
        job.weights[YVEX_MOE_WEIGHT_ROUTER] =
            ref_view(YVEX_GGUF_QTYPE_F32, (const unsigned char *)L->router, L->experts, L->hidden);
    } else {
        identity = (float *)calloc((size_t)(L->experts * L->experts), sizeof(float));
        if (!identity) return YVEX_ERR_NOMEM;
        for (e = 0; e < L->experts; ++e) identity[e * L->experts + e] = 1.0f;
        job.weights[YVEX_MOE_WEIGHT_ROUTER] =
            ref_view(YVEX_GGUF_QTYPE_F32, (const unsigned char *)identity, L->experts, width);
    }
    job.weights[YVEX_MOE_WEIGHT_ROUTER_BIAS] = ref_view(
        YVEX_GGUF_QTYPE_F32, (const unsigned char *)(L->bias ? L->bias : zero_bias), 1, L->experts);
    job.weights[YVEX_MOE_WEIGHT_ROUTER_TABLE] =
        ref_view(YVEX_GGUF_QTYPE_I32, (const unsigned char *)L->hash_table,
                 L->hash_stored_rows ? L->hash_stored_rows : 1, L->topk);
    rc = yvex_moe_route_cpu(&job, x_or_logits, &result, &err);
    free(identity);
    if (rc != YVEX_OK) return rc;
    for (e = 0; e < L->topk; ++e) {
        selected[e] = result.selected_experts[e];
        weights[e] = result.selected_weights[e];
    }
    if (logits) memcpy(logits, result.router_logits, (size_t)L->experts * sizeof(float));
    if (scores) memcpy(scores, result.router_scores, (size_t)L->experts * sizeof(float));
    return YVEX_OK;
}

/* One expert (gate/up/down given as single-expert row packs) on one bf16-rounded input row. */
int ref_expert(unsigned long long hidden, unsigned long long inter, double limit,
               unsigned int gate_qtype, unsigned int up_qtype, unsigned int down_qtype,
               const unsigned char *gate, const unsigned char *up, const unsigned char *down,
               const float *input, float route_weight, float *output) {
    yvex_moe_layer_plan plan;
    yvex_moe_weight_view g = ref_view(gate_qtype, gate, inter, hidden);
    yvex_moe_weight_view u = ref_view(up_qtype, up, inter, hidden);
    yvex_moe_weight_view d = ref_view(down_qtype, down, hidden, inter);
    yvex_error err;
    memset(&err, 0, sizeof(err));
    memset(&plan, 0, sizeof(plan));
    plan.hidden_width = hidden;
    plan.activation_limit = limit;
    return yvex_moe_expert_cpu(&plan, &g, &u, &d, input, route_weight, output, &err);
}

static int ref_round_bf16(float *v, unsigned long long n) {
    unsigned long long i;
    for (i = 0; i < n; ++i) {
        if (!isfinite(v[i])) return 0;
        v[i] = yvex_quant_bf16_decode(yvex_quant_bf16_encode(v[i]));
    }
    return 1;
}

/*
 * One token through route -> k routed experts (rank order, f32 adds) -> shared expert ->
 * bf16(routed + shared), as src/runtime/moe.c:596-632 does after the ingress step. `x` is the
 * hidden row BEFORE ingress rounding; it is bf16-rounded here like the normalized row the
 * reference feeds its router and experts (src/graph/moe.c:487-489).
 */
int ref_moe_token(const ref_moe_layer *L, const float *x, const float *logits,
                  unsigned int token_id, float *combined, float *routed_out, float *shared_out,
                  unsigned long long *selected, float *weights) {
    unsigned long long H = L->hidden, r, i;
    unsigned long long gate_rb = ref_row_bytes(L->gate_qtype, H);
    unsigned long long up_rb = ref_row_bytes(L->up_qtype, H);
    unsigned long long down_rb = ref_row_bytes(L->down_qtype, L->inter);
    float *xin = (float *)malloc((size_t)H * sizeof(float) * 4);
    float *routed, *shared, *expert;
    int rc;
    if (!xin) return YVEX_ERR_NOMEM;
    routed = xin + H;
    shared = routed + H;
    expert = shared + H;
    memcpy(xin, x, (size_t)H * sizeof(float));
    if (!ref_round_bf16(xin, H)) { free(xin); return YVEX_ERR_FORMAT; }
    rc = ref_route(L, L->router ? xin : logits, token_id, 1, selected, weights, NULL, NULL);
    memset(routed, 0, (size_t)H * sizeof(float));
    for (r = 0; rc == YVEX_OK && r < L->topk; ++r) {
        unsigned long long e = selected[r];
        rc = ref_expert(H, L->inter, L->limit, L->gate_qtype, L->up_qtype, L->down_qtype,
                        L->gate + e * L->inter * gate_rb, L->up + e * L->inter * up_rb,
                        L->down + e * H * down_rb, xin, weights[r], expert);
        if (rc == YVEX_OK)
            for (i = 0; i < H; ++i) routed[i] += expert[i];
    }
    if (rc == YVEX_OK)
        rc = ref_expert(H, L->shared_inter, L->limit, L->gate_qtype, L->up_qtype, L->down_qtype,
                        L->shared_gate, L->shared_up, L->shared_down, xin, 1.0f, shared);
    if (rc == YVEX_OK) {
        for (i = 0; i < H; ++i) combined[i] = routed[i] + shared[i];
        if (!ref_round_bf16(combined, H)) rc = YVEX_ERR_FORMAT;
        if (routed_out) memcpy(routed_out, routed, (size_t)H * sizeof(float));
        if (shared_out) memcpy(shared_out, shared, (size_t)H * sizeof(float));
    }
    free(xin);
    return rc;
}

typedef struct {
    const ref_moe_layer *L;
    const float *x, *logits;
    const unsigned int *token_ids;
    float *combined;
    unsigned long long *selected;
    float *weights;
    unsigned long long begin, end;
    int rc;
} ref_token_span;

static void *ref_token_worker(void *arg) {
    ref_token_span *s = (ref_token_span *)arg;
    unsigned long long t;
    for (t = s->begin; t < s->end; ++t) {
        int rc = ref_moe_token(s->L, s->x + t * s->L->hidden,
                               s->logits ? s->logits + t * s->L->experts : NULL,
                               s->token_ids ? s->token_ids[t] : 0u,
                               s->combined + t * s->L->hidden, NULL, NULL,
                               s->selected + t * s->L->topk, s->weights + t * s->L->topk);
        if (rc != YVEX_OK) { s->rc = rc; return NULL; }
    }
    return NULL;
}

/* `tokens` independent rows, split over `threads` pthreads (the CPU functions are re-entrant). */
int ref_moe_tokens(const ref_moe_layer *L, unsigned long long tokens, const float *x,
                   const float *logits, const unsigned int *token_ids, float *combined,
                   unsigned long long *selected, float *weights, int threads) {
    ref_token_span spans[REF_MAX_THREADS];
    pthread_t tids[REF_MAX_THREADS];
    int t, rc = YVEX_OK;
    if (threads < 1) threads = 1;
    if (threads > REF_MAX_THREADS) threads = REF_MAX_THREADS;
    if ((unsigned long long)threads > tokens) threads = (int)tokens;
    for (t = 0; t < threads; ++t) {
        spans[t] = (ref_token_span){L, x, logits, token_ids, combined, selected, weights,
                                    tokens * t / threads, tokens * (t + 1) / threads, YVEX_OK};
        if (threads == 1) ref_token_worker(&spans[t]);
        else if (pthread_create(&tids[t], NULL, ref_token_worker, &spans[t])) return YVEX_ERR;
    }
    for (t = 0; t < threads; ++t) {
        if (threads > 1) pthread_join(tids[t], NULL);
        if (spans[t].rc != YVEX_OK) rc = spans[t].rc;
    }
    return rc;
}

/* ---- mHC envelope of the MoE FFN ----------------------------------------------------------- */
typedef struct {
    unsigned long long hidden, streams, sinkhorn_iterations;
    double rms_epsilon, mhc_epsilon, post_multiplier;
    const float *mhc_fn, *scale, *base, *norm;
} ref_mhc;

static void ref_mhc_plan(const ref_mhc *M, yvex_moe_layer_plan *plan) {
    memset(plan, 0, sizeof(*plan));
    plan->hidden_width = M->hidden;
    plan->residual_streams = M->streams;
    plan->expanded_width = M->streams * M->hidden;
    plan->mhc_mixing_rows = (M->streams + 2ull) * M->streams;
    plan->mhc_sinkhorn_iterations = M->sinkhorn_iterations;
    plan->rms_epsilon = M->rms_epsilon;
    plan->mhc_epsilon = M->mhc_epsilon;
    plan->mhc_post_multiplier = M->post_multiplier;
}

/* yvex_moe_ffn_prepare_cpu (src/graph/moe.c:446-495): expanded row -> normalized FFN input,
 * post gates and the Sinkhorn-normalised stream combination. */
int ref_mhc_prepare(const ref_mhc *M, const float *expanded, float *normalized, float *post,
                    float *combination) {
    yvex_moe_layer_plan plan;
    yvex_moe_layer_job job;
    yvex_error err;
    memset(&err, 0, sizeof(err));
    memset(&job, 0, sizeof(job));
    ref_mhc_plan(M, &plan);
    job.layer = &plan;
    job.expanded_input = expanded;
    job.weights[YVEX_MOE_WEIGHT_MHC_FUNCTION] = ref_view(
        YVEX_GGUF_QTYPE_F32, (const unsigned char *)M->mhc_fn, plan.mhc_mixing_rows, plan.expanded_width);
    job.weights[YVEX_MOE_WEIGHT_MHC_SCALE] = ref_view(YVEX_GGUF_QTYPE_F32, (const unsigned char *)M->scale, 1, 3);
    job.weights[YVEX_MOE_WEIGHT_MHC_BASE] =
        ref_view(YVEX_GGUF_QTYPE_F32, (const unsigned char *)M->base, 1, plan.mhc_mixing_rows);
    job.weights[YVEX_MOE_WEIGHT_FFN_NORM] = ref_view(YVEX_GGUF_QTYPE_F32, (const unsigned char *)M->norm, 1, M->hidden);
    return yvex_moe_ffn_prepare_cpu(&job, normalized, post, combination, &err);
}

/* yvex_attention_mhc_post (src/graph/numeric.c:826-875) with the geometry the MoE FFN uses. */
int ref_mhc_post(const ref_mhc *M, const float *core, const float *expanded, const float *post,
                 const float *combination, float *out) {
    yvex_attention_layer_plan geometry;
    yvex_attention_mhc_post_args args;
    yvex_attention_failure failure;
    yvex_error err;
    const unsigned long long S = M->streams, H = M->hidden;
    memset(&err, 0, sizeof(err));
    memset(&failure, 0, sizeof(failure));
    memset(&geometry, 0, sizeof(geometry));
    geometry.compute_contract = YVEX_ATTENTION_COMPUTE_BF16_F32_RNE_V1;
    geometry.residual_stream_count = S;
    geometry.residual_stream_width = H;
    geometry.residual_expanded_width = S * H;
    geometry.mhc_mixing_rows = (S + 2ull) * S;
    geometry.mhc_mixing_columns = S * H;
    geometry.mhc_base_width = (S + 2ull) * S;
    geometry.mhc_scale_width = 3ull;
    geometry.mhc_sinkhorn_iterations = M->sinkhorn_iterations;
    geometry.rms_norm_epsilon = M->rms_epsilon;
    geometry.mhc_epsilon = M->mhc_epsilon;
    geometry.mhc_residual_post_multiplier = M->post_multiplier;
    geometry.mhc_attention_pre_and_post = 1;
    args = (yvex_attention_mhc_post_args){&geometry, core, expanded, post, combination, 1ull, H, S * H, S, S * S, out, S * H};
    return yvex_attention_mhc_post(&args, &failure, &err);
}

/* One attention head through the reference's public op on its CPU backend. */
int ref_attention_head(const float *q, const float *keys, const float *values,
                       unsigned long long seq_len, unsigned long long head_dim,
                       unsigned long long position, float scale, int causal, float *out) {
    yvex_backend *backend = NULL;
    yvex_device_tensor *tq = NULL, *tk = NULL, *tv = NULL, *ts = NULL, *tp = NULL, *to = NULL;
    yvex_backend_tensor_desc d;
    yvex_error err;
    int rc;
    memset(&err, 0, sizeof(err));
    rc = yvex_backend_open_cpu(&backend, &err);
    if (rc != YVEX_OK) return rc;
#define REF_ALLOC(t, nm, rk, d0, d1)                                                  \
    do {                                                                              \
        memset(&d, 0, sizeof(d));                                                     \
        d.name = nm; d.dtype = YVEX_DTYPE_F32; d.rank = rk; d.dims[0] = d0;           \
        d.dims[1] = d1; d.bytes = (unsigned long long)(d0) * ((rk) == 2 ? (d1) : 1ull) * 4ull; \
        if (rc == YVEX_OK) rc = yvex_backend_tensor_alloc(backend, &d, &t, &err);     \
    } while (0)
    REF_ALLOC(tq, "q", 1, head_dim, 0);
    REF_ALLOC(tk, "k", 2, seq_len, head_dim);
    REF_ALLOC(tv, "v", 2, seq_len, head_dim);
    REF_ALLOC(ts, "s", 1, seq_len, 0);
    REF_ALLOC(tp, "p", 1, seq_len, 0);
    REF_ALLOC(to, "o", 1, head_dim, 0);
#undef REF_ALLOC
    if (rc == YVEX_OK) rc = yvex_backend_tensor_write(backend, tq, q, head_dim * 4ull, &err);
    if (rc == YVEX_OK) rc = yvex_backend_tensor_write(backend, tk, keys, seq_len * head_dim * 4ull, &err);
    if (rc == YVEX_OK) rc = yvex_backend_tensor_write(backend, tv, values, seq_len * head_dim * 4ull, &err);
    if (rc == YVEX_OK)
        rc = yvex_backend_op_attention(backend, tq, tk, tv, seq_len, position, scale, causal, ts,
                                       tp, to, &err);
    if (rc == YVEX_OK) rc = yvex_backend_tensor_read(backend, to, out, head_dim * 4ull, &err);
    if (tq) yvex_backend_tensor_free(backend, tq);
    if (tk) yvex_backend_tensor_free(backend, tk);
    if (tv) yvex_backend_tensor_free(backend, tv);
    if (ts) yvex_backend_tensor_free(backend, ts);
    if (tp) yvex_backend_tensor_free(backend, tp);
    if (to) yvex_backend_tensor_free(backend, to);
    yvex_backend_close(backend);
    return rc;
}

/* ---- external MoE input fixture, sealed and serialized by the reference itself ------------------- */

/* Builds a fixture of `layers` layers (layer index 3 * ordinal + 1, the given widths) over `tokens`
 * tokens, has the reference seal it and write it to `path` (which must not exist). */
int ref_moe_input_write(const char *path, unsigned long long token_start, unsigned long long tokens,
                        unsigned long long layers, const unsigned long long *widths, const float *activations,
                        const unsigned int *token_ids) {
    yvex_moe_input_summary summary;
    yvex_moe_input_layer_record records[16];
    yvex_error err;
    unsigned long long offset = 0, i;
    static const char *ids[5] = {
        "1111111111111111111111111111111111111111111111111111111111111111",
        "2222222222222222222222222222222222222222222222222222222222222222",
        "3333333333333333333333333333333333333333333333333333333333333333",
        "4444444444444444444444444444444444444444444444444444444444444444",
        "abcdefabcdefabcdefabcdefabcdefabcdefabcdefabcdefabcdefabcdefabcd"};
    if (layers > 16) return YVEX_ERR_BOUNDS;
    memset(&summary, 0, sizeof(summary));
    memset(records, 0, sizeof(records));
    summary.schema_version = YVEX_MOE_INPUT_SCHEMA_V1;
    summary.token_start = token_start;
    summary.token_count = tokens;
    summary.layer_count = layers;
    summary.token_id_payload_bytes = tokens * sizeof(unsigned int);
    memcpy(summary.logical_model_identity, ids[0], 65);
    memcpy(summary.runtime_numeric_identity, ids[1], 65);
    memcpy(summary.runtime_descriptor_identity, ids[2], 65);
    memcpy(summary.moe_plan_identity, ids[3], 65);
    for (i = 0; i < layers; ++i) {
        records[i].ordinal = i;
        records[i].layer_index = 3 * i + 1;
        records[i].width = records[i].stride = widths[i];
        records[i].payload_offset = offset;
        records[i].payload_bytes = tokens * widths[i] * sizeof(float);
        memcpy(records[i].layer_identity, ids[4], 65);
        offset += records[i].payload_bytes;
    }
    summary.activation_payload_bytes = offset;
    int rc = yvex_moe_input_seal(&summary, records, activations, token_ids, &err);
    if (rc != YVEX_OK) return rc;
    return yvex_moe_input_write(path, &summary, records, activations, token_ids, &err);
}
