/*
 * TEST INFRASTRUCTURE - CPU restatement of the reference's quantized MoE hot path (see
 * yvex_oracle.h for scope and parity status). Written from the reference's behaviour, one
 * function per reference function, each citing the file:line it follows. Double accumulation,
 * float stores and bf16 rounding points are kept exactly where the reference has them because
 * results are compared bit-for-bit.
 */
#include "yvex_oracle.h"
#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

#define OQ_MAX_THREADS 256

/* ---- scalar codecs: src/gguf/quant_scalar.c:40-68 (f16), :123-143 (bf16) ------------------- */

static float oq_bits_float(uint32_t bits) {
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

float oq_f16_decode(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 31u, m = h & 1023u;
    if (e == 31u) return oq_bits_float(sign | 0x7f800000u | (m << 13) | (m ? 0x00400000u : 0u));
    if (e) return oq_bits_float(sign | ((e + 112u) << 23) | (m << 13));
    if (!m) return oq_bits_float(sign);
    { /* subnormal half: renormalise */
        uint32_t shift = 0;
        while (!(m & 1024u)) { m <<= 1; ++shift; }
        return oq_bits_float(sign | ((113u - shift) << 23) | ((m & 1023u) << 13));
    }
}

uint16_t oq_bf16_encode(float value) {
    uint32_t bits, hi, lo;
    memcpy(&bits, &value, 4);
    hi = bits >> 16;
    lo = bits & 0xffffu;
    if ((bits & 0x7f800000u) == 0x7f800000u && (bits & 0x007fffffu)) return (uint16_t)(hi | 0x40u);
    if (lo > 0x8000u || (lo == 0x8000u && (hi & 1u))) ++hi;
    return (uint16_t)hi;
}

float oq_bf16_decode(uint16_t bits) { return oq_bits_float((uint32_t)bits << 16); }
float oq_bf16_round(float v) { return oq_bf16_decode(oq_bf16_encode(v)); }

static uint16_t ld16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }
static uint32_t ld32(const uint8_t *p) {
    return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
}

/* ---- geometry and capability: src/gguf/qtype.c:15-104, src/gguf/quant_registry.c:50-103 ---- */

static const struct { uint16_t elems, bytes; } oq_geom[43] = {
    {1, 4},     {1, 2},     {32, 18},   {32, 20},   {0, 0},     {0, 0},    {32, 22},  {32, 24},
    {32, 34},   {32, 36},   {256, 84},  {256, 110}, {256, 144}, {256, 176}, {256, 210}, {256, 292},
    {256, 66},  {256, 74},  {256, 98},  {256, 50},  {32, 18},   {256, 110}, {256, 82}, {256, 136},
    {1, 1},     {1, 2},     {1, 4},     {1, 8},     {1, 8},     {256, 56},  {1, 2},    {0, 0},
    {0, 0},     {0, 0},     {256, 54},  {256, 66},  {0, 0},     {0, 0},     {0, 0},    {32, 17},
    {64, 36},   {128, 18},  {64, 18}};

int oq_geometry(unsigned qtype, unsigned *elems, unsigned *bytes) {
    if (qtype > 42u) return 0;
    if (elems) *elems = oq_geom[qtype].elems;
    if (bytes) *bytes = oq_geom[qtype].bytes;
    return 1;
}

int oq_capability(unsigned qtype, int allow_q4k) {
    if (qtype > 42u) return -1;
    switch (qtype) {
    case OQ_F32: case OQ_F16: case OQ_Q8_0: case OQ_Q2_K: case OQ_IQ2_XXS: case OQ_I32:
    case OQ_BF16: case OQ_MXFP4:
        return 31;
    case OQ_Q4_K:
        return allow_q4k ? (1 | 4 | 8 | 16) : 1;
    default:
        /* removed ids 4,5,31-33,36-38 and outside-baseline ids 40-42 have no storage either */
        return (oq_geom[qtype].elems && qtype < 40u) ? 1 : 0;
    }
}

/* ---- block decoders ------------------------------------------------------------------------ */

static const uint16_t oq_iq2_grid[256] = {
#include "iq2xxs_grid.inc"
};

/* src/gguf/quant_block.c:745-767 with the sign-parity rule of :378-386. */
static void oq_decode_iq2_xxs(const uint8_t *b, float *out) {
    float d = oq_f16_decode(ld16(b));
    for (unsigned g = 0; g < 8; ++g) {
        uint32_t idx = ld32(b + 2 + 8 * g), ss = ld32(b + 6 + 8 * g);
        float gs = d * (0.5f + (float)(ss >> 28)) * 0.25f;
        for (unsigned s = 0; s < 4; ++s) {
            uint16_t digits = oq_iq2_grid[(idx >> (8 * s)) & 255u];
            uint32_t low = (ss >> (7 * s)) & 127u, par = low;
            par ^= par >> 4; par ^= par >> 2; par ^= par >> 1;
            low |= (par & 1u) << 7;
            for (unsigned l = 0; l < 8; ++l) {
                unsigned digit = (digits >> (2 * l)) & 3u;
                float level = digit == 0 ? 8.0f : digit == 1 ? 25.0f : 43.0f;
                out[32 * g + 8 * s + l] = gs * level * ((low >> l) & 1u ? -1.0f : 1.0f);
            }
        }
    }
}

/* src/gguf/quant_block.c:715-743. */
static void oq_decode_q2_k(const uint8_t *b, float *out) {
    float d = oq_f16_decode(ld16(b + 80)), dmin = oq_f16_decode(ld16(b + 82));
    for (unsigned sub = 0; sub < 16; ++sub) {
        unsigned half = sub >> 3, plane = (sub >> 1) & 3u, pair = sub & 1u;
        const uint8_t *q = b + 16 + 32 * half + 16 * pair;
        float scale = d * (float)(b[sub] & 15u), minimum = dmin * (float)(b[sub] >> 4);
        for (unsigned l = 0; l < 16; ++l)
            out[16 * sub + l] = scale * (float)((q[l] >> (2 * plane)) & 3u) - minimum;
    }
}

/*
 * Q4_K, this repository's extension (no reference decoder exists; parity unpinned). Public GGUF
 * description: f16 d at 0, f16 dmin at 2, twelve bytes of 6-bit packed (scale, min) pairs for
 * eight 32-element sub-blocks at 4, 128 bytes of 4-bit codes at 16; sub-blocks 2p and 2p+1 share
 * 32 code bytes (low / high nibbles); value = (d*sc)*code - (dmin*m), evaluated in f32.
 */
static void oq_q4k_scale_min(const uint8_t *s, unsigned j, unsigned *sc, unsigned *m) {
    if (j < 4) { *sc = s[j] & 63u; *m = s[j + 4] & 63u; }
    else { *sc = (s[j + 4] & 15u) | ((s[j - 4] >> 6) << 4); *m = (s[j + 4] >> 4) | ((s[j] >> 6) << 4); }
}
static void oq_decode_q4_k(const uint8_t *b, float *out) {
    float d = oq_f16_decode(ld16(b)), dmin = oq_f16_decode(ld16(b + 2));
    for (unsigned j = 0; j < 8; ++j) {
        unsigned sc, m;
        const uint8_t *q = b + 16 + 32 * (j >> 1);
        oq_q4k_scale_min(b + 4, j, &sc, &m);
        float scale = d * (float)sc, minimum = dmin * (float)m;
        for (unsigned l = 0; l < 32; ++l)
            out[32 * j + l] = scale * (float)((j & 1u) ? q[l] >> 4 : q[l] & 15u) - minimum;
    }
}

static const float oq_mxfp4_levels[16] = {0.0f, 1.0f, 2.0f, 3.0f, 4.0f, 6.0f, 8.0f, 12.0f,
                                          -0.0f, -1.0f, -2.0f, -3.0f, -4.0f, -6.0f, -8.0f, -12.0f};

/* src/gguf/quant_block.c:769-881: exact-size check, scale sanity, fail-closed default. */
int oq_decode_block(unsigned qtype, const uint8_t *b, size_t bytes, float *out, size_t elements,
                    int allow_q4k) {
    int cap = oq_capability(qtype, allow_q4k);
    float d, dmin;
    if (!b || !out) return OQ_ERR_INVALID_ARG;
    if (cap < 0 || !(cap & 4)) return OQ_ERR_UNSUPPORTED;
    if (bytes != oq_geom[qtype].bytes || elements != oq_geom[qtype].elems) return OQ_ERR_FORMAT;
    switch (qtype) {
    case OQ_F32: out[0] = oq_bits_float(ld32(b)); return OQ_OK;
    case OQ_F16: out[0] = oq_f16_decode(ld16(b)); return OQ_OK;
    case OQ_BF16: out[0] = oq_bf16_decode(ld16(b)); return OQ_OK;
    case OQ_I32: out[0] = (float)(int32_t)ld32(b); return OQ_OK;
    case OQ_Q8_0:
        d = oq_f16_decode(ld16(b));
        if (!isfinite(d) || d < 0.0f) return OQ_ERR_FORMAT;
        for (unsigned i = 0; i < 32; ++i) out[i] = d * (float)(int8_t)b[2 + i];
        return OQ_OK;
    case OQ_MXFP4: {
        float scale;
        if (b[0] == 0xffu) return OQ_ERR_FORMAT;
        scale = oq_bits_float(b[0] ? (uint32_t)b[0] << 23 : 0x00400000u) * 0.5f;
        for (unsigned i = 0; i < 16; ++i) {
            out[i] = oq_mxfp4_levels[b[1 + i] & 15u] * scale;
            out[i + 16] = oq_mxfp4_levels[b[1 + i] >> 4] * scale;
            if (!isfinite(out[i]) || !isfinite(out[i + 16])) return OQ_ERR_FORMAT;
        }
        return OQ_OK;
    }
    case OQ_Q2_K:
        d = oq_f16_decode(ld16(b + 80));
        dmin = oq_f16_decode(ld16(b + 82));
        if (!isfinite(d) || !isfinite(dmin) || d < 0.0f || dmin < 0.0f) return OQ_ERR_FORMAT;
        oq_decode_q2_k(b, out);
        return OQ_OK;
    case OQ_Q4_K:
        d = oq_f16_decode(ld16(b));
        dmin = oq_f16_decode(ld16(b + 2));
        if (!isfinite(d) || !isfinite(dmin) || d < 0.0f || dmin < 0.0f) return OQ_ERR_FORMAT;
        oq_decode_q4_k(b, out);
        return OQ_OK;
    case OQ_IQ2_XXS:
        d = oq_f16_decode(ld16(b));
        if (!isfinite(d) || d < 0.0f) return OQ_ERR_FORMAT;
        oq_decode_iq2_xxs(b, out);
        return OQ_OK;
    default:
        return OQ_ERR_UNSUPPORTED;
    }
}

int oq_decode_rows(unsigned qtype, const uint8_t *encoded, uint64_t rows, uint64_t width,
                   float *out, int allow_q4k) {
    unsigned be, bb;
    if (!oq_geometry(qtype, &be, &bb) || !be || width % be) return OQ_ERR_BOUNDS;
    for (uint64_t blk = 0, n = rows * (width / be); blk < n; ++blk) {
        int rc = oq_decode_block(qtype, encoded + blk * bb, bb, out + blk * be, be, allow_q4k);
        if (rc != OQ_OK) return rc;
    }
    return OQ_OK;
}

/* src/gguf/quant_compute.c:116-181: per-block decode, sequential double accumulate, refusals. */
int oq_dot(unsigned qtype, const uint8_t *encoded, size_t bytes, const float *x,
           uint64_t elements, float *out, int allow_q4k) {
    int cap = oq_capability(qtype, allow_q4k);
    unsigned be, bb;
    double sum = 0.0;
    float values[256];
    if (!encoded || !x || !out || !elements) return OQ_ERR_INVALID_ARG;
    if (cap < 0 || !(cap & 8) || !oq_geometry(qtype, &be, &bb) || !be) return OQ_ERR_UNSUPPORTED;
    if (elements % be) return OQ_ERR_BOUNDS;
    if (elements / be * bb != bytes) return OQ_ERR_BOUNDS;
    for (uint64_t blk = 0; blk < elements / be; ++blk) {
        int rc = oq_decode_block(qtype, encoded + blk * bb, bb, values, be, allow_q4k);
        if (rc != OQ_OK) return rc;
        for (unsigned l = 0; l < be; ++l) {
            double term = (double)values[l] * x[blk * be + l];
            if (!isfinite(term) || !isfinite(sum + term)) return OQ_ERR_FORMAT;
            sum += term;
        }
    }
    *out = (float)sum;
    return isfinite(*out) ? OQ_OK : OQ_ERR_BOUNDS;
}

typedef struct {
    unsigned qtype; const uint8_t *w; uint64_t r0, r1, width, row_bytes; const float *x; float *y;
    int allow, rc;
} oq_mv_span;

static void *oq_mv_worker(void *arg) {
    oq_mv_span *s = (oq_mv_span *)arg;
    for (uint64_t r = s->r0; r < s->r1 && s->rc == OQ_OK; ++r)
        s->rc = oq_dot(s->qtype, s->w + r * s->row_bytes, (size_t)s->row_bytes, s->x, s->width,
                       &s->y[r], s->allow);
    return NULL;
}

/* src/graph/moe.c:430-444 (loop of row dots), optionally split over threads. */
int oq_matvec(unsigned qtype, const uint8_t *w, uint64_t rows, uint64_t width, const float *x,
              float *y, int threads, int allow_q4k) {
    oq_mv_span spans[OQ_MAX_THREADS];
    pthread_t tid[OQ_MAX_THREADS];
    unsigned be, bb;
    int rc = OQ_OK;
    if (!oq_geometry(qtype, &be, &bb) || !be) return OQ_ERR_UNSUPPORTED;
    if (width % be) return OQ_ERR_BOUNDS;
    if (threads < 1) threads = 1;
    if (threads > OQ_MAX_THREADS) threads = OQ_MAX_THREADS;
    for (int t = 0; t < threads; ++t) {
        spans[t] = (oq_mv_span){qtype, w, rows * t / threads, rows * (t + 1) / threads, width,
                                width / be * bb, x, y, allow_q4k, OQ_OK};
        if (threads == 1) oq_mv_worker(&spans[t]);
        else if (pthread_create(&tid[t], NULL, oq_mv_worker, &spans[t])) return -1;
    }
    for (int t = 0; t < threads; ++t) {
        if (threads > 1) pthread_join(tid[t], NULL);
        if (spans[t].rc != OQ_OK) rc = spans[t].rc;
    }
    return rc;
}

/* ---- router: src/graph/moe.c:497-585 --------------------------------------------------------- */

static double oq_sqrt_softplus(double v) {
    return sqrt(v > 0.0 ? v + log1p(exp(-v)) : log1p(exp(v)));
}

int oq_route(const oq_moe_layer *L, const float *x_or_logits, uint32_t token_id,
             int token_present, uint64_t *selected, float *weights, float *logits_out,
             float *scores_out) {
    float logits[256], scores[256], biased[256];
    double total = 0.0;
    if (!L || !x_or_logits || !selected || !weights || L->experts > 256 || L->topk > 16 ||
        L->topk > L->experts)
        return OQ_ERR_INVALID_ARG;
    for (uint64_t e = 0; e < L->experts; ++e) {
        if (L->router) {
            int rc = oq_dot(OQ_F32, (const uint8_t *)(L->router + e * L->hidden),
                            (size_t)L->hidden * 4, x_or_logits, L->hidden, &logits[e], 0);
            if (rc != OQ_OK) return rc;
        } else {
            if (!isfinite(x_or_logits[e])) return OQ_ERR_FORMAT;
            logits[e] = x_or_logits[e];
        }
        double s = oq_sqrt_softplus(logits[e]);
        if (!isfinite(s)) return OQ_ERR_FORMAT;
        scores[e] = (float)s;
    }
    if (L->router_class == 0) {
        if (!token_present || token_id >= L->hash_rows || !L->hash_table) return OQ_ERR_BOUNDS;
        for (uint64_t r = 0; r < L->topk; ++r) {
            int32_t e = L->hash_table[(L->hash_stored_rows == 1 ? 0 : (uint64_t)token_id * L->topk) + r];
            if (e < 0 || (uint64_t)e >= L->experts) return OQ_ERR_FORMAT;
            selected[r] = (uint64_t)e;
        }
    } else {
        for (uint64_t e = 0; e < L->experts; ++e)
            biased[e] = (L->bias ? L->bias[e] : 0.0f) + scores[e];
        for (uint64_t r = 0; r < L->topk; ++r) { /* k passes of arg-max; ties -> lower index */
            uint64_t best = UINT64_MAX;
            for (uint64_t e = 0; e < L->experts; ++e) {
                int used = 0;
                for (uint64_t p = 0; p < r; ++p) used |= selected[p] == e;
                if (!used && (best == UINT64_MAX || biased[e] > biased[best])) best = e;
            }
            selected[r] = best;
        }
    }
    for (uint64_t r = 0; r < L->topk; ++r) {
        for (uint64_t p = 0; p < r; ++p)
            if (selected[p] == selected[r]) return OQ_ERR_FORMAT;
        weights[r] = scores[selected[r]];
        total += weights[r];
    }
    if (L->normalize && (!isfinite(total) || total <= 0.0)) return OQ_ERR_FORMAT;
    for (uint64_t r = 0; r < L->topk; ++r) {
        double v = weights[r];
        if (L->normalize) v /= total;
        weights[r] = (float)(v * L->scaling);
    }
    if (logits_out) memcpy(logits_out, logits, (size_t)L->experts * 4);
    if (scores_out) memcpy(scores_out, scores, (size_t)L->experts * 4);
    return OQ_OK;
}

/* ---- expert: src/graph/moe.c:587-622 ---------------------------------------------------------- */

static uint64_t oq_row_bytes(unsigned qtype, uint64_t width) {
    unsigned be, bb;
    return oq_geometry(qtype, &be, &bb) && be ? width / be * bb : 0;
}

int oq_expert(uint64_t H, uint64_t I, double limit, unsigned gq, unsigned uq, unsigned dq,
              const uint8_t *gate, const uint8_t *up, const uint8_t *down, const float *input,
              float route_weight, float *output, int allow) {
    float g[4096], u[4096], mid[4096];
    int rc;
    if (!gate || !up || !down || !input || !output || !isfinite(route_weight))
        return OQ_ERR_INVALID_ARG;
    if (I > 4096) return OQ_ERR_BOUNDS;
    if ((rc = oq_matvec(gq, gate, I, H, input, g, 1, allow)) != OQ_OK) return rc;
    if ((rc = oq_matvec(uq, up, I, H, input, u, 1, allow)) != OQ_OK) return rc;
    for (uint64_t i = 0; i < I; ++i) {
        double gv = fmin(g[i], limit), uv = fmax(-limit, fmin(u[i], limit));
        double silu = gv >= 0.0 ? gv / (1.0 + exp(-gv)) : gv * exp(gv) / (1.0 + exp(gv));
        mid[i] = (float)(silu * uv * route_weight);
        if (!isfinite(mid[i])) return OQ_ERR_FORMAT;
        mid[i] = oq_bf16_round(mid[i]);
    }
    if ((rc = oq_matvec(dq, down, H, I, mid, output, 1, allow)) != OQ_OK) return rc;
    for (uint64_t i = 0; i < H; ++i) {
        if (!isfinite(output[i])) return OQ_ERR_FORMAT;
        output[i] = oq_bf16_round(output[i]);
    }
    return OQ_OK;
}

/* ---- layer: src/runtime/moe.c:596-632 after the ingress rounding of src/graph/moe.c:487-489 --- */

int oq_moe_token(const oq_moe_layer *L, const float *x, const float *logits, uint32_t token_id,
                 float *combined, float *routed_out, float *shared_out, uint64_t *selected,
                 float *weights) {
    uint64_t H = L->hidden;
    uint64_t grb = oq_row_bytes(L->gate_qtype, H), urb = oq_row_bytes(L->up_qtype, H);
    uint64_t drb = oq_row_bytes(L->down_qtype, L->inter);
    float *buf = (float *)malloc((size_t)H * 4 * sizeof(float));
    float *xin = buf, *routed = buf + H, *shared = buf + 2 * H, *one = buf + 3 * H;
    int rc;
    if (!buf) return OQ_ERR_NOMEM;
    for (uint64_t i = 0; i < H; ++i) {
        if (!isfinite(x[i])) { free(buf); return OQ_ERR_FORMAT; }
        xin[i] = oq_bf16_round(x[i]);
    }
    rc = oq_route(L, L->router ? xin : logits, token_id, 1, selected, weights, NULL, NULL);
    memset(routed, 0, (size_t)H * sizeof(float));
    for (uint64_t r = 0; rc == OQ_OK && r < L->topk; ++r) {
        uint64_t e = selected[r];
        rc = oq_expert(H, L->inter, L->limit, L->gate_qtype, L->up_qtype, L->down_qtype,
                       L->gate + e * L->inter * grb, L->up + e * L->inter * urb,
                       L->down + e * H * drb, xin, weights[r], one, L->allow_q4k);
        for (uint64_t i = 0; rc == OQ_OK && i < H; ++i) routed[i] += one[i];
    }
    if (rc == OQ_OK)
        rc = oq_expert(H, L->shared_inter, L->limit, L->gate_qtype, L->up_qtype, L->down_qtype,
                       L->shared_gate, L->shared_up, L->shared_down, xin, 1.0f, shared,
                       L->allow_q4k);
    for (uint64_t i = 0; rc == OQ_OK && i < H; ++i) {
        combined[i] = routed[i] + shared[i];
        if (!isfinite(combined[i])) rc = OQ_ERR_FORMAT;
        else combined[i] = oq_bf16_round(combined[i]);
    }
    if (rc == OQ_OK && routed_out) memcpy(routed_out, routed, (size_t)H * 4);
    if (rc == OQ_OK && shared_out) memcpy(shared_out, shared, (size_t)H * 4);
    free(buf);
    return rc;
}

typedef struct {
    const oq_moe_layer *L; const float *x, *logits; const uint32_t *ids; float *combined;
    uint64_t *selected; float *weights; uint64_t t0, t1; int rc;
} oq_tok_span;

static void *oq_tok_worker(void *arg) {
    oq_tok_span *s = (oq_tok_span *)arg;
    const oq_moe_layer *L = s->L;
    for (uint64_t t = s->t0; t < s->t1 && s->rc == OQ_OK; ++t)
        s->rc = oq_moe_token(L, s->x + t * L->hidden, s->logits ? s->logits + t * L->experts : NULL,
                             s->ids ? s->ids[t] : 0u, s->combined + t * L->hidden, NULL, NULL,
                             s->selected + t * L->topk, s->weights + t * L->topk);
    return NULL;
}

int oq_moe_tokens(const oq_moe_layer *L, uint64_t tokens, const float *x, const float *logits,
                  const uint32_t *ids, float *combined, uint64_t *selected, float *weights,
                  int threads) {
    oq_tok_span spans[OQ_MAX_THREADS];
    pthread_t tid[OQ_MAX_THREADS];
    int rc = OQ_OK;
    if (threads < 1) threads = 1;
    if (threads > OQ_MAX_THREADS) threads = OQ_MAX_THREADS;
    if ((uint64_t)threads > tokens) threads = (int)tokens;
    for (int t = 0; t < threads; ++t) {
        spans[t] = (oq_tok_span){L, x, logits, ids, combined, selected, weights,
                                 tokens * t / threads, tokens * (t + 1) / threads, OQ_OK};
        if (threads == 1) oq_tok_worker(&spans[t]);
        else if (pthread_create(&tid[t], NULL, oq_tok_worker, &spans[t])) return -1;
    }
    for (int t = 0; t < threads; ++t) {
        if (threads > 1) pthread_join(tid[t], NULL);
        if (spans[t].rc != OQ_OK) rc = spans[t].rc;
    }
    return rc;
}

/* ---- mHC envelope: src/graph/moe.c:446-495, src/graph/numeric.c:630-659,694-875 -------------- */

static double oq_sigmoid(double v) {                          /* numeric.c:694-704 */
    if (v >= 0.0) return 1.0 / (1.0 + exp(-v));
    double d = exp(v);
    return d / (1.0 + d);
}

static int oq_sinkhorn(float *m, uint64_t n, uint64_t iterations, double eps) {   /* numeric.c:706-750 */
    for (uint64_t r = 0; r < n; ++r) {
        double mx = -(double)INFINITY, total = 0.0;
        for (uint64_t c = 0; c < n; ++c) mx = fmax(mx, m[r * n + c]);
        for (uint64_t c = 0; c < n; ++c) {
            double v = exp((double)m[r * n + c] - mx);
            m[r * n + c] = (float)v;
            total += v;
        }
        if (!isfinite(total) || total <= 0.0) return 0;
        for (uint64_t c = 0; c < n; ++c) m[r * n + c] = (float)((double)m[r * n + c] / total + eps);
    }
    for (uint64_t it = 0; it < iterations; ++it) {
        if (it != 0) {
            for (uint64_t r = 0; r < n; ++r) {
                double total = 0.0;
                for (uint64_t c = 0; c < n; ++c) total += m[r * n + c];
                if (!isfinite(total)) return 0;
                for (uint64_t c = 0; c < n; ++c) m[r * n + c] = (float)((double)m[r * n + c] / (total + eps));
            }
        }
        for (uint64_t c = 0; c < n; ++c) {
            double total = 0.0;
            for (uint64_t r = 0; r < n; ++r) total += m[r * n + c];
            if (!isfinite(total)) return 0;
            for (uint64_t r = 0; r < n; ++r) m[r * n + c] = (float)((double)m[r * n + c] / (total + eps));
        }
    }
    return 1;
}

int oq_mhc_prepare(const oq_mhc *M, const float *expanded, float *normalized, float *post,
                   float *combination) {
    const uint64_t S = M->streams, H = M->hidden, W = S * H, rows = (S + 2) * S;
    float mix[64];
    if (!S || !H || rows > 64 || H > 16384) return OQ_ERR_INVALID_ARG;        /* moe.c:455-457 */
    int rc = oq_matvec(OQ_F32, (const uint8_t *)M->mhc_fn, rows, W, expanded, mix, 1, 0);
    if (rc != OQ_OK) return rc;
    for (uint64_t i = 0; i < 3; ++i) if (!isfinite(M->scale[i])) return OQ_ERR_FORMAT;
    for (uint64_t i = 0; i < rows; ++i) if (!isfinite(M->base[i])) return OQ_ERR_FORMAT;
    double squares = 0.0;
    memset(normalized, 0, (size_t)H * sizeof(float));
    for (uint64_t i = 0; i < W; ++i) {
        if (!isfinite(expanded[i])) return OQ_ERR_FORMAT;
        squares += (double)expanded[i] * (double)expanded[i];
    }
    double inv = 1.0 / sqrt(squares / (double)W + M->rms_epsilon);
    if (!isfinite(inv)) return OQ_ERR_FORMAT;
    for (uint64_t s = 0; s < S; ++s) {                                        /* numeric.c:794-813 */
        double pre = oq_sigmoid((double)mix[s] * inv * (double)M->scale[0] + (double)M->base[s]);
        post[s] = (float)(M->post_multiplier *
                          oq_sigmoid((double)mix[S + s] * inv * (double)M->scale[1] + (double)M->base[S + s]));
        for (uint64_t t = 0; t < S; ++t) {
            uint64_t idx = 2 * S + s * S + t;
            combination[s * S + t] = (float)((double)mix[idx] * inv * (double)M->scale[2] + (double)M->base[idx]);
        }
        for (uint64_t i = 0; i < H; ++i)
            normalized[i] += (float)((pre + M->mhc_epsilon) * (double)expanded[s * H + i]);
    }
    if (!oq_sinkhorn(combination, S, M->sinkhorn_iterations, M->mhc_epsilon)) return OQ_ERR_FORMAT;
    for (uint64_t i = 0; i < H; ++i) {
        if (!isfinite(normalized[i])) return OQ_ERR_FORMAT;
        normalized[i] = oq_bf16_round(normalized[i]);
    }
    double mean = 0.0;                                                        /* numeric.c:630-659 */
    for (uint64_t i = 0; i < H; ++i) {
        if (!isfinite(M->norm[i])) return OQ_ERR_FORMAT;
        mean += (double)normalized[i] * (double)normalized[i];
    }
    mean /= (double)H;
    double ninv = 1.0 / sqrt(mean + M->rms_epsilon);
    if (!isfinite(ninv)) return OQ_ERR_FORMAT;
    for (uint64_t i = 0; i < H; ++i) {
        double v = (double)normalized[i] * ninv * (double)M->norm[i];
        if (!isfinite(v)) return OQ_ERR_FORMAT;
        normalized[i] = oq_bf16_round((float)v);
    }
    return OQ_OK;
}

int oq_mhc_post(const oq_mhc *M, const float *core, const float *expanded, const float *post,
                const float *combination, float *out) {                       /* numeric.c:826-875 */
    const uint64_t S = M->streams, H = M->hidden;
    for (uint64_t t = 0; t < S; ++t)
        for (uint64_t i = 0; i < H; ++i) {
            double v = (double)post[t] * (double)core[i];
            for (uint64_t s = 0; s < S; ++s) v += (double)combination[s * S + t] * (double)expanded[s * H + i];
            if (!isfinite(v)) return OQ_ERR_FORMAT;
            out[t * H + i] = oq_bf16_round((float)v);
        }
    return OQ_OK;
}

/* ---- expert worklist: src/graph/worklist.c:369-441 ------------------------------------------- */

int oq_worklist(const uint64_t *selected, uint64_t rows, uint64_t topk, uint64_t experts,
                uint32_t *order, uint32_t *source_rows, uint32_t *bucket_expert,
                uint32_t *bucket_offset, uint32_t *bucket_count, uint32_t *bucket_total) {
    uint64_t pairs = rows * topk, cursor = 0, buckets = 0;
    for (uint64_t e = 0; e < experts; ++e) {
        uint64_t start = cursor;
        for (uint64_t p = 0; p < pairs; ++p) {
            if (selected[p] >= experts) return OQ_ERR_FORMAT;
            if (selected[p] != e) continue;
            order[cursor] = (uint32_t)p;        /* source pair == destination row */
            source_rows[cursor] = (uint32_t)(p / topk);
            ++cursor;
        }
        if (cursor == start) continue;           /* only populated experts get a bucket */
        bucket_expert[buckets] = (uint32_t)e;
        bucket_offset[buckets] = (uint32_t)start;
        bucket_count[buckets] = (uint32_t)(cursor - start);
        ++buckets;
    }
    bucket_offset[buckets] = (uint32_t)cursor;
    *bucket_total = (uint32_t)buckets;
    return cursor == pairs ? OQ_OK : OQ_ERR_FORMAT;
}

/* ---- attention: src/backend/cpu.c:229-267 (range-reduced Taylor exp) and :319-411 ------------- */

static double oq_exp_taylor(double x) {
    const double ln2 = 0.69314718055994530942;
    double term = 1.0, sum = 1.0;
    int n = 0;
    if (x < -60.0) return 0.0;
    if (x > 60.0) x = 60.0;
    while (x > 0.5) { x -= ln2; ++n; }
    while (x < -0.5) { x += ln2; --n; }
    for (unsigned i = 1; i <= 18; ++i) { term *= x / (double)i; sum += term; }
    for (; n > 0; --n) sum *= 2.0;
    for (; n < 0; ++n) sum *= 0.5;
    return sum;
}

int oq_attention_head(const float *q, const float *keys, const float *values, uint64_t seq_len,
                      uint64_t head_dim, uint64_t position, float scale, int causal, float *out) {
    uint64_t visible = causal ? position + 1 : seq_len;
    double max_score = 0.0, sum = 0.0;
    float *score, *prob;
    if (!isfinite(scale) || scale <= 0.0f) return OQ_ERR_INVALID_ARG;
    if (!seq_len || !head_dim) return OQ_ERR_FORMAT;
    if (position >= seq_len) return OQ_ERR_BOUNDS;
    score = (float *)malloc((size_t)seq_len * 2 * sizeof(float));
    if (!score) return OQ_ERR_NOMEM;
    prob = score + seq_len;
    for (uint64_t i = 0; i < visible; ++i) {
        double s = 0.0;
        for (uint64_t d = 0; d < head_dim; ++d) s += (double)q[d] * (double)keys[i * head_dim + d];
        s *= (double)scale;
        score[i] = (float)s;                   /* the max uses the unrounded double score */
        if (i == 0 || s > max_score) max_score = s;
    }
    for (uint64_t i = 0; i < visible; ++i) {
        double e = oq_exp_taylor((double)score[i] - max_score);
        prob[i] = (float)e;
        sum += e;
    }
    if (sum <= 0.0) { free(score); return -8; }
    for (uint64_t i = 0; i < visible; ++i) prob[i] = (float)((double)prob[i] / sum);
    for (uint64_t d = 0; d < head_dim; ++d) {
        double v = 0.0;
        for (uint64_t i = 0; i < visible; ++i) v += (double)prob[i] * (double)values[i * head_dim + d];
        out[d] = (float)v;
    }
    free(score);
    return OQ_OK;
}

typedef struct {
    const uint16_t *q, *k, *v; uint64_t q_heads, kv_heads, context, dim, position; float scale;
    float *out; uint64_t h0, h1; int rc;
} oq_att_span;

static void *oq_att_worker(void *arg) {
    oq_att_span *s = (oq_att_span *)arg;
    uint64_t n = s->context * s->dim, group = s->q_heads / s->kv_heads;
    float *kf = (float *)malloc((size_t)(2 * n + s->dim) * sizeof(float));
    if (!kf) { s->rc = OQ_ERR_NOMEM; return NULL; }
    float *vf = kf + n, *qf = vf + n;
    uint64_t cached = UINT64_MAX;
    for (uint64_t h = s->h0; h < s->h1 && s->rc == OQ_OK; ++h) {
        uint64_t session = h / s->q_heads, head = h % s->q_heads;
        uint64_t kv = session * s->kv_heads + head / group;
        if (kv != cached) {
            for (uint64_t i = 0; i < n; ++i) {
                kf[i] = oq_bf16_decode(s->k[kv * n + i]);
                vf[i] = oq_bf16_decode(s->v[kv * n + i]);
            }
            cached = kv;
        }
        for (uint64_t d = 0; d < s->dim; ++d) qf[d] = oq_bf16_decode(s->q[h * s->dim + d]);
        s->rc = oq_attention_head(qf, kf, vf, s->context, s->dim, s->position, s->scale, 1,
                                  s->out + h * s->dim);
    }
    free(kf);
    return NULL;
}

int oq_attention_gqa_decode(const uint16_t *q, const uint16_t *k, const uint16_t *v,
                            uint64_t sessions, uint64_t q_heads, uint64_t kv_heads,
                            uint64_t context, uint64_t head_dim, uint64_t position, float scale,
                            float *out, int threads) {
    oq_att_span spans[OQ_MAX_THREADS];
    pthread_t tid[OQ_MAX_THREADS];
    uint64_t heads = sessions * q_heads;
    int rc = OQ_OK;
    if (!kv_heads || q_heads % kv_heads) return OQ_ERR_INVALID_ARG;
    if (threads < 1) threads = 1;
    if (threads > OQ_MAX_THREADS) threads = OQ_MAX_THREADS;
    if ((uint64_t)threads > heads) threads = (int)heads;
    for (int t = 0; t < threads; ++t) {
        spans[t] = (oq_att_span){q, k, v, q_heads, kv_heads, context, head_dim, position, scale,
                                 out, heads * t / threads, heads * (t + 1) / threads, OQ_OK};
        if (threads == 1) oq_att_worker(&spans[t]);
        else if (pthread_create(&tid[t], NULL, oq_att_worker, &spans[t])) return -1;
    }
    for (int t = 0; t < threads; ++t) {
        if (threads > 1) pthread_join(tid[t], NULL);
        if (spans[t].rc != OQ_OK) rc = spans[t].rc;
    }
    return rc;
}
