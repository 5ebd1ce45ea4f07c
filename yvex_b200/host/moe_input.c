/*
 * Reader of the reference's external MoE input fixtures (files named *.yvex-moe-input), so that the
 * same activation files can drive this backend's MoE operators unchanged.
 *
 * Format (src/runtime/moe_input.c:30-36, :226-277, all integers little-endian u64):
 *   [0, 16)    magic "YVEXMOEINPUT001\0"
 *   [16, 64)   schema version (1), token start, token count, layer count, activation payload bytes,
 *              token id payload bytes
 *   [64, 512)  seven 64-character lowercase-hex identities: logical model, runtime numeric, runtime
 *              descriptor, MoE plan, activation payload digest, token id payload digest, input identity
 *   then       one 112-byte record per layer: ordinal, layer index, width, stride, payload offset,
 *              payload bytes, 64-character layer identity
 *   then       the activation payload (f32, layer after layer, [token count x width] each)
 *   then       the token ids (u32)
 * Admission follows the reference (:145-196, :279-357): exact total size (trailing bytes are a
 * format error, a short file a bounds error), ordinals in order, stride == width, contiguous
 * ranges, no duplicate layer, finite activations, both payload digests (SHA-256) and the
 * path-independent input identity must match. Files must be regular, not symbolic links, and within
 * the caller's size bound.
 */
#define _GNU_SOURCE
#include "backend_private.h"

#include <errno.h>
#include <fcntl.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/stat.h>
#include <unistd.h>

#define INPUT_HEADER_BYTES 512ull
#define INPUT_RECORD_BYTES 112ull
#define INPUT_MAX_LAYERS 1024ull

static const unsigned char input_magic[16] = {'Y', 'V', 'E', 'X', 'M', 'O', 'E', 'I', 'N', 'P', 'U', 'T', '0', '0', '1', '\0'};

struct yvex_moe_input {
    yvex_moe_input_summary summary;
    yvex_moe_input_layer_record *records;
    unsigned char *bytes;                  /* the whole image, owned */
    size_t byte_count;
    const float *activations;
    const unsigned int *token_ids;
};

/* ---- SHA-256 (FIPS 180-4) ----------------------------------------------------------------------- */
typedef struct { uint32_t h[8]; unsigned char block[64]; uint64_t total; size_t fill; } sha256;

static const uint32_t sha_k[64] = {
    0x428a2f98u, 0x71374491u, 0xb5c0fbcfu, 0xe9b5dba5u, 0x3956c25bu, 0x59f111f1u, 0x923f82a4u, 0xab1c5ed5u, 0xd807aa98u, 0x12835b01u,
    0x243185beu, 0x550c7dc3u, 0x72be5d74u, 0x80deb1feu, 0x9bdc06a7u, 0xc19bf174u, 0xe49b69c1u, 0xefbe4786u, 0x0fc19dc6u, 0x240ca1ccu,
    0x2de92c6fu, 0x4a7484aau, 0x5cb0a9dcu, 0x76f988dau, 0x983e5152u, 0xa831c66du, 0xb00327c8u, 0xbf597fc7u, 0xc6e00bf3u, 0xd5a79147u,
    0x06ca6351u, 0x14292967u, 0x27b70a85u, 0x2e1b2138u, 0x4d2c6dfcu, 0x53380d13u, 0x650a7354u, 0x766a0abbu, 0x81c2c92eu, 0x92722c85u,
    0xa2bfe8a1u, 0xa81a664bu, 0xc24b8b70u, 0xc76c51a3u, 0xd192e819u, 0xd6990624u, 0xf40e3585u, 0x106aa070u, 0x19a4c116u, 0x1e376c08u,
    0x2748774cu, 0x34b0bcb5u, 0x391c0cb3u, 0x4ed8aa4au, 0x5b9cca4fu, 0x682e6ff3u, 0x748f82eeu, 0x78a5636fu, 0x84c87814u, 0x8cc70208u,
    0x90befffau, 0xa4506cebu, 0xbef9a3f7u, 0xc67178f2u};

static uint32_t rotr(uint32_t v, unsigned n) { return (v >> n) | (v << (32u - n)); }

static void sha_block(sha256 *s, const unsigned char *p) {
    uint32_t w[64], a, b, c, d, e, f, g, h;
    for (int i = 0; i < 16; ++i) w[i] = (uint32_t)p[4 * i] << 24 | (uint32_t)p[4 * i + 1] << 16 | (uint32_t)p[4 * i + 2] << 8 | p[4 * i + 3];
    for (int i = 16; i < 64; ++i) {
        const uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
        const uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
        w[i] = w[i - 16] + s0 + w[i - 7] + s1;
    }
    a = s->h[0]; b = s->h[1]; c = s->h[2]; d = s->h[3]; e = s->h[4]; f = s->h[5]; g = s->h[6]; h = s->h[7];
    for (int i = 0; i < 64; ++i) {
        const uint32_t t1 = h + (rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25)) + ((e & f) ^ (~e & g)) + sha_k[i] + w[i];
        const uint32_t t2 = (rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22)) + ((a & b) ^ (a & c) ^ (b & c));
        h = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
    }
    s->h[0] += a; s->h[1] += b; s->h[2] += c; s->h[3] += d; s->h[4] += e; s->h[5] += f; s->h[6] += g; s->h[7] += h;
}

static void sha_init(sha256 *s) {
    static const uint32_t iv[8] = {0x6a09e667u, 0xbb67ae85u, 0x3c6ef372u, 0xa54ff53au, 0x510e527fu, 0x9b05688cu, 0x1f83d9abu, 0x5be0cd19u};
    memcpy(s->h, iv, sizeof(iv));
    s->total = 0; s->fill = 0;
}

static void sha_update(sha256 *s, const void *data, size_t n) {
    const unsigned char *p = (const unsigned char *)data;
    s->total += n;
    while (n) {
        size_t take = 64u - s->fill;
        if (take > n) take = n;
        memcpy(s->block + s->fill, p, take);
        s->fill += take; p += take; n -= take;
        if (s->fill == 64u) { sha_block(s, s->block); s->fill = 0; }
    }
}

/* u64 as eight little-endian bytes; text as its length (u64) followed by its bytes: the reference's
 * identity encoding (src/core/sha256.c:185-203). */
static void sha_u64(sha256 *s, unsigned long long v) {
    unsigned char b[8];
    for (int i = 0; i < 8; ++i) b[i] = (unsigned char)(v >> (8 * i));
    sha_update(s, b, 8);
}

static void sha_text(sha256 *s, const char *text) {
    const size_t n = text ? strlen(text) : 0u;
    sha_u64(s, n);
    sha_update(s, text, n);
}

static void sha_hex(sha256 *s, char out[YVEX_SHA256_HEX_CAP]) {
    const uint64_t bits = s->total * 8u;
    unsigned char pad[72] = {0x80};
    const size_t padn = (s->fill < 56u ? 56u : 120u) - s->fill;
    for (int i = 0; i < 8; ++i) pad[padn + i] = (unsigned char)(bits >> (56 - 8 * i));
    sha_update(s, pad, padn + 8u);
    for (int i = 0; i < 8; ++i) snprintf(out + 8 * i, 9, "%08x", s->h[i]);
    out[64] = 0;
}

/* ---- admission ------------------------------------------------------------------------------------ */
static int refuse(yvex_error *err, yvex_status code, const char *why) { return yvex_refuse(err, code, "runtime.moe-input", why); }

static unsigned long long get_u64(const unsigned char *p) {
    unsigned long long v = 0;
    for (int i = 0; i < 8; ++i) v |= (unsigned long long)p[i] << (8 * i);
    return v;
}

static int hex_valid(const char *id) {
    if (!id) return 0;
    for (int i = 0; i < 64; ++i)
        if (!((id[i] >= '0' && id[i] <= '9') || (id[i] >= 'a' && id[i] <= 'f'))) return 0;
    return id[64] == 0;
}

static int mul_ok(unsigned long long a, unsigned long long b, unsigned long long *out) { return !__builtin_mul_overflow(a, b, out); }
static int add_ok(unsigned long long a, unsigned long long b, unsigned long long *out) { return !__builtin_add_overflow(a, b, out); }

static void input_identity(const yvex_moe_input_summary *s, const yvex_moe_input_layer_record *r, char out[YVEX_SHA256_HEX_CAP]) {
    sha256 h;
    sha_init(&h);
    sha_text(&h, "yvex.runtime.moe-input.v1");
    sha_u64(&h, s->schema_version); sha_u64(&h, s->token_start); sha_u64(&h, s->token_count); sha_u64(&h, s->layer_count);
    sha_u64(&h, s->activation_payload_bytes); sha_u64(&h, s->token_id_payload_bytes);
    sha_text(&h, s->logical_model_identity); sha_text(&h, s->runtime_numeric_identity); sha_text(&h, s->runtime_descriptor_identity);
    sha_text(&h, s->moe_plan_identity); sha_text(&h, s->activation_payload_digest); sha_text(&h, s->token_id_payload_digest);
    for (unsigned long long i = 0; i < s->layer_count; ++i) {
        sha_u64(&h, r[i].ordinal); sha_u64(&h, r[i].layer_index); sha_u64(&h, r[i].width); sha_u64(&h, r[i].stride);
        sha_u64(&h, r[i].payload_offset); sha_u64(&h, r[i].payload_bytes);
        sha_text(&h, r[i].layer_identity);
    }
    sha_hex(&h, out);
}

/* Parses and verifies an image the input now owns. */
static int admit(yvex_moe_input *in, yvex_error *err) {
    yvex_moe_input_summary *s = &in->summary;
    const unsigned char *b = in->bytes, *cur;
    unsigned long long records_bytes, act_off, tok_off, total, offset = 0, token_bytes;
    char digest[YVEX_SHA256_HEX_CAP];
    sha256 h;
    if (in->byte_count < INPUT_HEADER_BYTES || memcmp(b, input_magic, sizeof(input_magic)) != 0)
        return refuse(err, YVEX_ERR_FORMAT, "MoE input magic or header is invalid");
    s->schema_version = (unsigned int)get_u64(b + 16);
    s->token_start = get_u64(b + 24); s->token_count = get_u64(b + 32); s->layer_count = get_u64(b + 40);
    s->activation_payload_bytes = get_u64(b + 48); s->token_id_payload_bytes = get_u64(b + 56);
    {
        char *ids[7] = {s->logical_model_identity, s->runtime_numeric_identity, s->runtime_descriptor_identity, s->moe_plan_identity,
                        s->activation_payload_digest, s->token_id_payload_digest, s->input_identity};
        for (int i = 0; i < 7; ++i) { memcpy(ids[i], b + 64 + 64 * i, 64); ids[i][64] = 0; }
    }
    if (s->schema_version != 1u || !s->token_count || !s->layer_count || !s->activation_payload_bytes || !s->token_id_payload_bytes ||
        !hex_valid(s->logical_model_identity) || !hex_valid(s->runtime_numeric_identity) || !hex_valid(s->runtime_descriptor_identity) ||
        !hex_valid(s->moe_plan_identity) || s->layer_count > INPUT_MAX_LAYERS || !mul_ok(s->layer_count, INPUT_RECORD_BYTES, &records_bytes) ||
        !add_ok(INPUT_HEADER_BYTES, records_bytes, &act_off) || !add_ok(act_off, s->activation_payload_bytes, &tok_off) ||
        !add_ok(tok_off, s->token_id_payload_bytes, &total) || total != in->byte_count) {
        const int trailing = s->schema_version == 1u && add_ok(INPUT_HEADER_BYTES, s->layer_count * INPUT_RECORD_BYTES, &act_off) &&
                             add_ok(act_off, s->activation_payload_bytes, &tok_off) && add_ok(tok_off, s->token_id_payload_bytes, &total) &&
                             total < in->byte_count;
        return refuse(err, trailing ? YVEX_ERR_FORMAT : YVEX_ERR_BOUNDS,
                      trailing ? "MoE input contains trailing bytes" : "MoE input is truncated or oversized");
    }
    in->records = (yvex_moe_input_layer_record *)calloc((size_t)s->layer_count, sizeof(*in->records));
    if (!in->records) return refuse(err, YVEX_ERR_NOMEM, "MoE input record allocation failed");
    cur = b + INPUT_HEADER_BYTES;
    for (unsigned long long i = 0; i < s->layer_count; ++i, cur += INPUT_RECORD_BYTES) {
        yvex_moe_input_layer_record *r = &in->records[i];
        r->ordinal = get_u64(cur); r->layer_index = get_u64(cur + 8); r->width = get_u64(cur + 16); r->stride = get_u64(cur + 24);
        r->payload_offset = get_u64(cur + 32); r->payload_bytes = get_u64(cur + 40);
        memcpy(r->layer_identity, cur + 48, 64);
        r->layer_identity[64] = 0;
    }
    in->activations = (const float *)(b + act_off);
    in->token_ids = (const unsigned int *)(b + tok_off);
    if (!mul_ok(s->token_count, 4ull, &token_bytes) || token_bytes != s->token_id_payload_bytes)
        return refuse(err, YVEX_ERR_INVALID_ARG, "complete canonical MoE input facts are required");
    for (unsigned long long i = 0; i < s->layer_count; ++i) {
        const yvex_moe_input_layer_record *r = &in->records[i];
        unsigned long long elements, bytes;
        if (r->ordinal != i || r->stride != r->width || !r->width || r->payload_offset != offset ||
            !mul_ok(s->token_count, r->stride, &elements) || !mul_ok(elements, 4ull, &bytes) || r->payload_bytes != bytes ||
            !add_ok(offset, bytes, &offset) || !hex_valid(r->layer_identity))
            return refuse(err, YVEX_ERR_FORMAT, "MoE input layer ordering or range is malformed");
        for (unsigned long long p = 0; p < i; ++p)
            if (in->records[p].layer_index == r->layer_index) return refuse(err, YVEX_ERR_FORMAT, "MoE input contains a duplicate layer");
    }
    if (offset != s->activation_payload_bytes) return refuse(err, YVEX_ERR_FORMAT, "MoE activation ranges are not exact and contiguous");
    for (unsigned long long i = 0; i < offset / 4ull; ++i)
        if (!isfinite(in->activations[i])) return refuse(err, YVEX_ERR_FORMAT, "MoE input contains a non-finite activation");
    sha_init(&h); sha_update(&h, in->activations, (size_t)s->activation_payload_bytes); sha_hex(&h, digest);
    if (strcmp(digest, s->activation_payload_digest) != 0) return refuse(err, YVEX_ERR_FORMAT, "MoE payload digest mismatch");
    sha_init(&h); sha_update(&h, in->token_ids, (size_t)s->token_id_payload_bytes); sha_hex(&h, digest);
    if (strcmp(digest, s->token_id_payload_digest) != 0) return refuse(err, YVEX_ERR_FORMAT, "MoE payload digest mismatch");
    input_identity(s, in->records, digest);
    if (strcmp(digest, s->input_identity) != 0) return refuse(err, YVEX_ERR_FORMAT, "MoE input identity mismatch");
    yvex_error_clear(err);
    return YVEX_OK;
}

void yvex_moe_input_close(yvex_moe_input **input) {
    if (!input || !*input) return;
    free((*input)->records);
    free((*input)->bytes);
    free(*input);
    *input = NULL;
}

int yvex_moe_input_open_image(yvex_moe_input **out, const void *image, unsigned long long bytes, yvex_error *err) {
    yvex_moe_input *in;
    int rc;
    if (out) *out = NULL;
    if (!out || !image || !bytes || bytes > (unsigned long long)SIZE_MAX) return refuse(err, YVEX_ERR_INVALID_ARG, "an image is required");
    in = (yvex_moe_input *)calloc(1, sizeof(*in));
    if (!in) return refuse(err, YVEX_ERR_NOMEM, "MoE input allocation failed");
    /* a private copy, 16-byte aligned, so the f32 and u32 views are aligned whatever the caller's buffer is */
    if (posix_memalign((void **)&in->bytes, 64, (size_t)bytes) != 0) { free(in); return refuse(err, YVEX_ERR_NOMEM, "MoE input allocation failed"); }
    memcpy(in->bytes, image, (size_t)bytes);
    in->byte_count = (size_t)bytes;
    rc = admit(in, err);
    if (rc != YVEX_OK) { yvex_moe_input_close(&in); return rc; }
    *out = in;
    return YVEX_OK;
}

int yvex_moe_input_open_file(yvex_moe_input **out, const char *path, const yvex_moe_input_limits *limits, yvex_error *err) {
    const unsigned long long maximum = limits ? limits->maximum_file_bytes : 0ull;
    struct stat st;
    unsigned char *buf = NULL;
    size_t got = 0;
    int fd, rc;
    if (out) *out = NULL;
    if (!out || !path || !path[0] || !maximum) return refuse(err, YVEX_ERR_INVALID_ARG, "bounded MoE tensor-file arguments are required");
    fd = open(path, O_RDONLY | O_NOFOLLOW | O_CLOEXEC);
    if (fd < 0 || fstat(fd, &st) != 0 || !S_ISREG(st.st_mode) || st.st_size <= 0) {
        if (fd >= 0) close(fd);
        return refuse(err, YVEX_ERR_IO, "MoE input is not a readable regular non-symlink file");
    }
    if ((unsigned long long)st.st_size > maximum) { close(fd); return refuse(err, YVEX_ERR_BOUNDS, "MoE input exceeds its resource bound"); }
    buf = (unsigned char *)malloc((size_t)st.st_size);
    if (!buf) { close(fd); return refuse(err, YVEX_ERR_NOMEM, "MoE input allocation failed"); }
    while (got < (size_t)st.st_size) {
        const ssize_t n = read(fd, buf + got, (size_t)st.st_size - got);
        if (n < 0 && errno == EINTR) continue;
        if (n <= 0) break;
        got += (size_t)n;
    }
    close(fd);
    if (got != (size_t)st.st_size) { free(buf); return refuse(err, YVEX_ERR_IO, "MoE input could not be read"); }
    rc = yvex_moe_input_open_image(out, buf, got, err);
    free(buf);
    return rc;
}

const yvex_moe_input_summary *yvex_moe_input_summary_get(const yvex_moe_input *input) { return input ? &input->summary : NULL; }

int yvex_moe_input_layer_view(const yvex_moe_input *input, unsigned long long ordinal, const float **values, unsigned long long *stride,
                              yvex_error *err) {
    if (values) *values = NULL;
    if (stride) *stride = 0;
    if (!input || !values || !stride) return refuse(err, YVEX_ERR_INVALID_ARG, "input, values and stride are required");
    if (ordinal >= input->summary.layer_count) return refuse(err, YVEX_ERR_BOUNDS, "MoE input layer ordinal is out of range");
    *values = input->activations + input->records[ordinal].payload_offset / 4ull;
    *stride = input->records[ordinal].stride;
    yvex_error_clear(err);
    return YVEX_OK;
}

const yvex_moe_input_layer_record *yvex_moe_input_layer_record_at(const yvex_moe_input *input, unsigned long long ordinal) {
    return input && ordinal < input->summary.layer_count ? &input->records[ordinal] : NULL;
}

const unsigned int *yvex_moe_input_token_ids(const yvex_moe_input *input) { return input ? input->token_ids : NULL; }

/* The fixture's rows of one layer as the row batch execute_rows / execute_rows_wide take (host rows). */
int yvex_moe_input_row_batch(const yvex_moe_input *input, unsigned long long ordinal, yvex_moe_row_batch *batch, yvex_error *err) {
    const float *values;
    unsigned long long stride;
    int rc;
    if (!batch) return refuse(err, YVEX_ERR_INVALID_ARG, "a row batch is required");
    memset(batch, 0, sizeof(*batch));
    rc = yvex_moe_input_layer_view(input, ordinal, &values, &stride, err);
    if (rc != YVEX_OK) return rc;
    batch->schema_version = YVEX_MOE_ROW_BATCH_SCHEMA_V1;
    batch->execution_class = YVEX_EXECUTION_CLASS_DEVICE_NATIVE;
    batch->provenance = input->summary.token_count > 1ull ? 3 : 0;      /* prefill rows, or a single row */
    batch->row_count = input->summary.token_count;
    batch->row_width = batch->row_stride = stride;
    batch->expanded_rows = values;
    batch->token_ids = input->token_ids;
    batch->token_ids_present = 1;
    return YVEX_OK;
}
