/*
 * TEST INFRASTRUCTURE - a plain-C, single-file CPU restatement of the reference's quantized MoE
 * hot path. It exists only to check the CUDA library: tests/, the smoke check and the CPU-baseline
 * legs of bench.py load it; the shipped library never does.
 *
 * Parity status: PINNED for F32/F16/BF16/Q8_0/Q2_K/IQ2_XXS decode, row dots, router, expert,
 * layer combine, worklist and single-head attention - tests/test_oracle.py checks this file
 * against the reference's own golden blocks and known answers and, where the compiled reference
 * (oracle/_ref) is present, bit-for-bit against it on seeded inputs; the same comparisons are
 * frozen in tests/golden/. Q4_K: PARITY UNPINNED - the reference admits Q4_K storage but ships no
 * decoder (src/gguf/quant_registry.c:67), so oq_decode_block's Q4_K branch restates the public
 * GGUF block description and is checked only for self-consistency.
 *
 * All status codes are the reference's yvex_status values (include/yvex/core.h:13-26).
 */
#ifndef YVEX_ORACLE_H
#define YVEX_ORACLE_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

enum { OQ_OK = 0, OQ_ERR_NOMEM = -2, OQ_ERR_FORMAT = -4, OQ_ERR_UNSUPPORTED = -5,
       OQ_ERR_BOUNDS = -7, OQ_ERR_INVALID_ARG = -10 };
enum { OQ_F32 = 0, OQ_F16 = 1, OQ_Q8_0 = 8, OQ_Q2_K = 10, OQ_Q4_K = 12, OQ_IQ2_XXS = 16,
       OQ_I32 = 26, OQ_BF16 = 30, OQ_MXFP4 = 39 };

float oq_f16_decode(uint16_t bits);
uint16_t oq_bf16_encode(float value);
float oq_bf16_decode(uint16_t bits);
float oq_bf16_round(float value);

/* Geometry (block elements / bytes) of every qtype id 0..42; returns 0 for unknown ids. */
int oq_geometry(unsigned qtype, unsigned *block_elements, unsigned *block_bytes);
/* Bit flags like the reference registry row: 1 storage, 4 decoder, 8 cpu dot, 16 device dot.
 * `allow_q4k` switches on this repository's Q4_K extension. */
int oq_capability(unsigned qtype, int allow_q4k);

int oq_decode_block(unsigned qtype, const uint8_t *encoded, size_t bytes, float *out,
                    size_t elements, int allow_q4k);
int oq_decode_rows(unsigned qtype, const uint8_t *encoded, uint64_t rows, uint64_t width,
                   float *out, int allow_q4k);
int oq_dot(unsigned qtype, const uint8_t *encoded, size_t bytes, const float *x,
           uint64_t elements, float *out, int allow_q4k);
int oq_matvec(unsigned qtype, const uint8_t *encoded, uint64_t rows, uint64_t width,
              const float *x, float *y, int threads, int allow_q4k);

typedef struct {
    uint64_t hidden, experts, topk, inter, shared_inter;
    double scaling, limit;
    int normalize, router_class; /* 1 learned hidden-state router, 0 token-id hash router */
    unsigned gate_qtype, up_qtype, down_qtype;
    const float *router;       /* [experts x hidden] f32; NULL => logits are supplied */
    const float *bias;         /* [experts] or NULL */
    const int32_t *hash_table; /* [hash_stored_rows x topk]; a single stored row serves every id */
    uint64_t hash_rows, hash_stored_rows;
    const uint8_t *gate, *up, *down; /* routed packs, expert-major */
    const uint8_t *shared_gate, *shared_up, *shared_down;
    int allow_q4k;
} oq_moe_layer;

int oq_route(const oq_moe_layer *L, const float *x_or_logits, uint32_t token_id,
             int token_present, uint64_t *selected, float *weights, float *logits, float *scores);
int oq_expert(uint64_t hidden, uint64_t inter, double limit, unsigned gate_qtype,
              unsigned up_qtype, unsigned down_qtype, const uint8_t *gate, const uint8_t *up,
              const uint8_t *down, const float *input, float route_weight, float *output,
              int allow_q4k);
int oq_moe_token(const oq_moe_layer *L, const float *x, const float *logits, uint32_t token_id,
                 float *combined, float *routed, float *shared, uint64_t *selected,
                 float *weights);
int oq_moe_tokens(const oq_moe_layer *L, uint64_t tokens, const float *x, const float *logits,
                  const uint32_t *token_ids, float *combined, uint64_t *selected, float *weights,
                  int threads);

/* ---- mHC envelope of the MoE FFN (4 residual streams around the layer) -------------------------
 * prepare: mix = mhc_fn . expanded (double dots), sigmoid gates, Sinkhorn-normalised stream
 * combination, collapse of the streams to one bf16-rounded row, RMSNorm * weight, bf16 round
 * (src/graph/moe.c:446-495, src/graph/numeric.c:630-659,694-824). post: re-expansion
 * out[t] = bf16(post[t]*core + sum_s combination[s][t]*residual[s]) (src/graph/numeric.c:826-875). */
typedef struct {
    uint64_t hidden, streams, sinkhorn_iterations;
    double rms_epsilon, mhc_epsilon, post_multiplier;
    const float *mhc_fn; /* [(streams + 2) * streams rows x streams * hidden] f32 */
    const float *scale;  /* [3] */
    const float *base;   /* [(streams + 2) * streams] */
    const float *norm;   /* [hidden] */
} oq_mhc;
int oq_mhc_prepare(const oq_mhc *M, const float *expanded, float *normalized, float *post,
                   float *combination);
int oq_mhc_post(const oq_mhc *M, const float *core, const float *expanded, const float *post,
                const float *combination, float *out);

/* Expert-major stable counting sort of (row, rank) pairs. Arrays sized pairs / experts(+1). */
int oq_worklist(const uint64_t *selected, uint64_t rows, uint64_t topk, uint64_t experts,
                uint32_t *order, uint32_t *source_rows, uint32_t *bucket_expert,
                uint32_t *bucket_offset, uint32_t *bucket_count, uint32_t *bucket_total);

int oq_attention_head(const float *q, const float *keys, const float *values, uint64_t seq_len,
                      uint64_t head_dim, uint64_t position, float scale, int causal, float *out);
/* GQA decode over a bf16 KV cache [sessions][kv_heads][context][head_dim]; one reference
 * single-head op per (session, q head), KV head = q head / (q_heads / kv_heads). */
int oq_attention_gqa_decode(const uint16_t *q_bf16, const uint16_t *k_bf16,
                            const uint16_t *v_bf16, uint64_t sessions, uint64_t q_heads,
                            uint64_t kv_heads, uint64_t context, uint64_t head_dim,
                            uint64_t position, float scale, float *out, int threads);
#ifdef __cplusplus
}
#endif
#endif
