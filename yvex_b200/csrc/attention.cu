// Online-softmax attention.
//
// gqa_decode: one query position per session against a bf16 KV cache. The cache is the only
// traffic that matters (2 x context x head_dim x 2 bytes per KV head), so the kernel is built to
// stream it once and to spend as few issue slots per key as possible: a CTA owns one (session,
// KV head) and one slice of the context; each warp walks 16-key blocks of the slice and does both
// contractions on the tensor cores (mma.sync m16n8k16, bf16 x bf16 -> f32):
//   S = Q K^T   M = heads of the GQA group (rows 0..G-1 of 16), N = 8 keys, K = 16 dims
//   O += P V    M = heads, K = 16 keys, N = 8 dims; P is split into hi + lo bf16 so the
//               probabilities keep ~16 mantissa bits
// Operands are built straight from coalesced 16-byte global loads without a shared-memory
// transpose: a dot product does not care in which order its terms are summed, so the k-slots of
// the MMA are assigned to whatever dims (for S) or keys (for O) a lane happens to hold, as long as
// both operands use the same assignment; the n-slots of O are a fixed permutation of the dims
// that the epilogue undoes. Scores stay in f32; the running (max, sum, accumulator) triple is
// rescaled once per 16-key block. Warps, then slices, are merged by log-sum-exp.
// Math per (session, q head) is the reference CPU op's: scores = scale * q.k, softmax over keys
// 0..position, out = sum p*v (src/backend/cpu.c:319-411).
#include <cuda_bf16.h>

#include "common.cuh"

namespace yb {

constexpr int kAttnThreads = 128;
constexpr int kAttnWarps = kAttnThreads / 32;
constexpr int kKeyBlock = 16;
constexpr int kMaxGroup = 8;                  // q heads per kv head that fit the 8 usable MMA rows

// D(16x8, f32) = A(16x16, bf16, row) * B(16x8, bf16, col) + C. Rows 8..15 of A are zero (a1 = a3 = 0):
// only d0, d1 (row lane/4) are kept.
__device__ __forceinline__ void mma_bf16_rows8(float &d0, float &d1, uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    float z0, z1;
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%10,%10};"
        : "+f"(d0), "+f"(d1), "=f"(z0), "=f"(z1)
        : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1), "f"(0.0f));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

__device__ __forceinline__ uint4 ldg_stream(const uint16_t *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// Partial layout per (session, kv head, split): G heads x (m, l, acc[D]).
template <int D>
__global__ void __launch_bounds__(kAttnThreads, 3)
gqa_decode_kernel(const uint16_t *__restrict__ q, const uint16_t *__restrict__ k,
                  const uint16_t *__restrict__ v, int kv_heads, int G, uint64_t context, uint64_t visible,
                  float scale, int splits, uint64_t keys_per_split, float *__restrict__ partial, int *status) {
    constexpr int KL = D / 32;                 // 16-byte K chunks a lane loads per key (chunks c, c+4, ...)
    constexpr int VU = D / 64;                 // 16-byte V chunks a lane loads per key (chunks g, g+8, ...)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, c = lane & 3;
    const int split = blockIdx.x % splits;
    const uint64_t sk = blockIdx.x / splits;           // session * kv_heads + kv head
    const uint64_t session = sk / kv_heads, kvh = sk % kv_heads;
    const uint16_t *kb = k + sk * context * D, *vb = v + sk * context * D;
    const uint16_t *qb = q + (session * (uint64_t)kv_heads * G + kvh * G) * D;

    // A fragments of Q: lane (g, c) holds head g, chunks c + 4i; rows >= G are zero.
    uint32_t qa[KL][4];
#pragma unroll
    for (int i = 0; i < KL; ++i) {
        uint4 raw = g < G ? __ldg(reinterpret_cast<const uint4 *>(qb + g * D) + c + 4 * i) : make_uint4(0, 0, 0, 0);
        qa[i][0] = raw.x; qa[i][1] = raw.y; qa[i][2] = raw.z; qa[i][3] = raw.w;
    }
    float m = -INFINITY, l = 0.0f;             // head g; l is this lane's share (4 keys of every 16)
    float acc[VU][8][2];                       // head g, dims 8*(2c + 8u) + 8*e + j  <-  acc[u][j][e]
#pragma unroll
    for (int u = 0; u < VU; ++u)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[u][j][0] = acc[u][j][1] = 0.0f;

    const uint64_t begin = (uint64_t)split * keys_per_split;
    const uint64_t end = begin + keys_per_split < visible ? begin + keys_per_split : visible;
    for (uint64_t base = begin + (uint64_t)warp * kKeyBlock; base < end; base += (uint64_t)kAttnWarps * kKeyBlock) {
        // ---- loads: K rows base+g and base+8+g (chunks c+4i); V rows base+{2c, 2c+1, 2c+8, 2c+9} (chunks g+8u)
        uint4 kr[2][KL], vr[4][VU];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const uint64_t key = base + 8 * half + g;
#pragma unroll
            for (int i = 0; i < KL; ++i)
                kr[half][i] = key < end ? ldg_stream(kb + key * D + 8 * (c + 4 * i)) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const uint64_t key = base + 2 * c + (r & 1) + 8 * (r >> 1);
#pragma unroll
            for (int u = 0; u < VU; ++u)
                vr[r][u] = key < end ? ldg_stream(vb + key * D + 8 * (g + 8 * u)) : make_uint4(0, 0, 0, 0);
        }
        // ---- S = Q K^T: sc[half][e] = score of head g, key base + 8*half + 2c + e
        float sc[2][2];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            sc[half][0] = sc[half][1] = 0.0f;
#pragma unroll
            for (int i = 0; i < KL; ++i) {
                const uint32_t w[4] = {kr[half][i].x, kr[half][i].y, kr[half][i].z, kr[half][i].w};
                mma_bf16_rows8(sc[half][0], sc[half][1], qa[i][0], qa[i][1], w[0], w[1]);
                mma_bf16_rows8(sc[half][0], sc[half][1], qa[i][2], qa[i][3], w[2], w[3]);
            }
        }
        float bm = m;
#pragma unroll
        for (int half = 0; half < 2; ++half)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const uint64_t key = base + 8 * half + 2 * c + e;
                sc[half][e] = key < end ? sc[half][e] * scale : -INFINITY;
                bm = fmaxf(bm, sc[half][e]);
            }
        bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
        bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 2));
        const float corr = __expf(m - bm);          // m = -inf on the first block -> 0
        m = bm;
        l *= corr;
        if (corr != 1.0f) {
#pragma unroll
            for (int u = 0; u < VU; ++u)
#pragma unroll
                for (int j = 0; j < 8; ++j) { acc[u][j][0] *= corr; acc[u][j][1] *= corr; }
        }
        // ---- P as A fragments (hi + lo bf16), keys 2c, 2c+1 (k-slots 2c..) and 2c+8, 2c+9 (k-slots 2c+8..)
        uint32_t ph[2], pl[2];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const float p0 = __expf(sc[half][0] - bm), p1 = __expf(sc[half][1] - bm);
            ph[half] = pack_bf16(p0, p1);
            const float r0 = p0 - __uint_as_float(ph[half] << 16), r1 = p1 - __uint_as_float(ph[half] & 0xffff0000u);
            pl[half] = pack_bf16(r0, r1);
            l += p0 + p1;
        }
        // ---- O += P V: n-tile (u, j) covers dim j of chunks 8u..8u+7; B pairs two keys of one dim
#pragma unroll
        for (int u = 0; u < VU; ++u) {
            const uint32_t r0[4] = {vr[0][u].x, vr[0][u].y, vr[0][u].z, vr[0][u].w};
            const uint32_t r1[4] = {vr[1][u].x, vr[1][u].y, vr[1][u].z, vr[1][u].w};
            const uint32_t r2[4] = {vr[2][u].x, vr[2][u].y, vr[2][u].z, vr[2][u].w};
            const uint32_t r3[4] = {vr[3][u].x, vr[3][u].y, vr[3][u].z, vr[3][u].w};
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t sel = (j & 1) ? 0x7632u : 0x5410u;
                const uint32_t b0 = __byte_perm(r0[j >> 1], r1[j >> 1], sel), b1 = __byte_perm(r2[j >> 1], r3[j >> 1], sel);
                mma_bf16_rows8(acc[u][j][0], acc[u][j][1], ph[0], ph[1], b0, b1);
                mma_bf16_rows8(acc[u][j][0], acc[u][j][1], pl[0], pl[1], b0, b1);
            }
        }
    }
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);

    // Merge the warps of the CTA through shared memory.
    __shared__ float sm_m[kAttnWarps][kMaxGroup], sm_l[kAttnWarps][kMaxGroup];
    __shared__ float sm_acc[kAttnWarps][kMaxGroup][D];
    if (g < G) {
        if (c == 0) { sm_m[warp][g] = m; sm_l[warp][g] = l; }
#pragma unroll
        for (int u = 0; u < VU; ++u)
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int e = 0; e < 2; ++e) sm_acc[warp][g][8 * (2 * c + e + 8 * u) + j] = acc[u][j][e];
    }
    __syncthreads();
    float *po = partial + ((sk * splits + split) * G) * (uint64_t)(D + 2);
    for (int idx = threadIdx.x; idx < G * D; idx += kAttnThreads) {
        const int h = idx / D, d = idx % D;
        float gm = -INFINITY;
        for (int w = 0; w < kAttnWarps; ++w) gm = fmaxf(gm, sm_m[w][h]);
        float gl = 0.0f, ga = 0.0f;
        for (int w = 0; w < kAttnWarps; ++w) {
            const float f = sm_m[w][h] == -INFINITY ? 0.0f : __expf(sm_m[w][h] - gm);
            gl += sm_l[w][h] * f;
            ga += sm_acc[w][h][d] * f;
        }
        if (d == 0) { po[h * (D + 2)] = gm; po[h * (D + 2) + 1] = gl; }
        po[h * (D + 2) + 2 + d] = ga;
    }
    (void)status;
}

template <int D, int G>
__global__ void gqa_merge_kernel(const float *__restrict__ partial, int splits, uint64_t groups,
                                 float *__restrict__ out, int *status) {
    // one CTA per (session, kv head); thread per (head, dim)
    const uint64_t sk = blockIdx.x;
    for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
        const int h = idx / D, d = idx % D;
        const float *p = partial + (sk * splits * G + h) * (uint64_t)(D + 2);
        float gm = -INFINITY;
        for (int s = 0; s < splits; ++s) gm = fmaxf(gm, p[(uint64_t)s * G * (D + 2)]);
        float gl = 0.0f, ga = 0.0f;
        for (int s = 0; s < splits; ++s) {
            const float *ps = p + (uint64_t)s * G * (D + 2);
            const float c = ps[0] == -INFINITY ? 0.0f : __expf(ps[0] - gm);
            gl += ps[1] * c;
            ga += ps[2 + d] * c;
        }
        const float o = ga / gl;
        if (!(gl > 0.0f) || !isfinite(o)) raise(status, YVEX_B200_STATUS_NUMERIC);
        out[(sk * G + h) * D + d] = o;
    }
    (void)groups;
}

// ---- the reference's public single-head op (f32 everything, scratch tensors written) ------------
__global__ void attention_f32_kernel(const float *q, const float *keys, const float *values, uint64_t seq_len,
                                     uint64_t D, uint64_t visible, float scale, float *scores, float *probs,
                                     float *out, int *status) {
    __shared__ float red[32];
    __shared__ float bcast;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (uint64_t i = warp; i < seq_len; i += nw) {
        if (i >= visible) { if (lane == 0) { scores[i] = 0.0f; probs[i] = 0.0f; } continue; }
        double s = 0.0;
        for (uint64_t d = lane; d < D; d += 32) s += (double)q[d] * (double)keys[i * D + d];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) scores[i] = (float)(s * (double)scale);
    }
    __syncthreads();
    float mx = -INFINITY;
    for (uint64_t i = threadIdx.x; i < visible; i += blockDim.x) mx = fmaxf(mx, scores[i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    if (threadIdx.x == 0) { float t = red[0]; for (int w = 1; w < nw; ++w) t = fmaxf(t, red[w]); bcast = t; }
    __syncthreads();
    mx = bcast;
    float sum = 0.0f;
    for (uint64_t i = threadIdx.x; i < visible; i += blockDim.x) {
        float e = expf(scores[i] - mx);
        probs[i] = e;
        sum += e;
    }
    sum = warp_sum(sum);
    __syncthreads();
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    if (threadIdx.x == 0) { float t = 0.0f; for (int w = 0; w < nw; ++w) t += red[w]; bcast = t; }
    __syncthreads();
    sum = bcast;
    if (!(sum > 0.0f)) { raise(status, YVEX_B200_STATUS_NUMERIC); return; }
    for (uint64_t i = threadIdx.x; i < visible; i += blockDim.x) probs[i] = probs[i] / sum;
    __syncthreads();
    for (uint64_t d = threadIdx.x; d < D; d += blockDim.x) {
        double a = 0.0;
        for (uint64_t i = 0; i < visible; ++i) a += (double)probs[i] * (double)values[i * D + d];
        out[d] = (float)a;
    }
}

// ---- sink reducer: every head of one token against one shared set of rows -----------------------
// The reference's reduce_head (src/graph/core.c:428-465) with reduce_visit_row (:318-345): the rows are key
// and value at once (one latent row set shared by all query heads), scores are f64 dot products times
// scale, the head's sink is the initial maximum and seeds the denominator with exp(sink - max), the
// output is sum p * row / denominator, optionally rounded to bf16. One CTA per head; a warp walks every
// kWarps-th row with a running maximum (f64), denominator (f64) and f32 partial sums, and the warps'
// states are merged through shared memory at the end (the reference makes two passes in row order; the
// results differ by f32 rounding only). D <= 1024.
constexpr int kSinkWarps = 8, kSinkMaxPerLane = 32;
__global__ void __launch_bounds__(32 * kSinkWarps) attention_sink_kernel(const float *query, const float *rows, const float *sinks, uint64_t n,
                                                                         uint64_t D, double scale, int round_bf16, float *out, int *status) {
    __shared__ double s_max[kSinkWarps], s_den[kSinkWarps];
    __shared__ float s_acc[kSinkWarps][1024];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint64_t head = blockIdx.x;
    const float *q = query + head * D;
    const int per_lane = (int)((D + 31) / 32);
    float qv[kSinkMaxPerLane], acc[kSinkMaxPerLane];
    bool bad = false;
#pragma unroll
    for (int j = 0; j < kSinkMaxPerLane; ++j) {
        const uint64_t d = (uint64_t)lane + 32u * j;
        qv[j] = j < per_lane && d < D ? q[d] : 0.0f;
        bad |= !isfinite(qv[j]);
        acc[j] = 0.0f;
    }
    const double sink = (double)sinks[head];
    bad |= !isfinite(sink);
    double mx = warp == 0 ? sink : -INFINITY, den = warp == 0 ? 1.0 : 0.0;      // the sink is a row without a value
    for (uint64_t i = warp; i < n; i += kSinkWarps) {
        const float *row = rows + i * D;
        float rv[kSinkMaxPerLane];
        double s = 0.0;
#pragma unroll
        for (int j = 0; j < kSinkMaxPerLane; ++j) {
            const uint64_t d = (uint64_t)lane + 32u * j;
            rv[j] = j < per_lane && d < D ? __ldg(row + d) : 0.0f;
            bad |= !isfinite(rv[j]);
            s += (double)qv[j] * (double)rv[j];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        s *= scale;
        bad |= !isfinite(s);
        if (s > mx) {
            const double c = exp(mx - s);                                   // 0 when nothing has been seen yet
            den *= c;
#pragma unroll
            for (int j = 0; j < kSinkMaxPerLane; ++j) acc[j] = (float)((double)acc[j] * c);
            mx = s;
        }
        const double p = exp(s - mx);
        den += p;
#pragma unroll
        for (int j = 0; j < kSinkMaxPerLane; ++j) acc[j] += (float)(p * (double)rv[j]);
    }
    if (lane == 0) { s_max[warp] = mx; s_den[warp] = den; }
#pragma unroll
    for (int j = 0; j < kSinkMaxPerLane; ++j)
        if (j < per_lane && (uint64_t)lane + 32u * j < D) s_acc[warp][lane + 32 * j] = acc[j];
    if (bad) raise(status, YVEX_B200_STATUS_NUMERIC);
    __syncthreads();
    double gm = s_max[0];
    for (int w = 1; w < kSinkWarps; ++w) gm = fmax(gm, s_max[w]);
    double gd = 0.0;
    for (int w = 0; w < kSinkWarps; ++w) gd += s_den[w] * (s_max[w] == -INFINITY ? 0.0 : exp(s_max[w] - gm));
    if (!(gd > 0.0) || !isfinite(gd)) { if (threadIdx.x == 0) raise(status, YVEX_B200_STATUS_NUMERIC); return; }
    for (uint64_t d = threadIdx.x; d < D; d += blockDim.x) {
        double a = 0.0;
        for (int w = 0; w < kSinkWarps; ++w) a += (double)s_acc[w][d] * (s_max[w] == -INFINITY ? 0.0 : exp(s_max[w] - gm));
        const float v = (float)(a / gd);
        if (!isfinite(v)) raise(status, YVEX_B200_STATUS_NUMERIC);
        out[head * D + d] = round_bf16 ? bf16_round(v) : v;
    }
}

static int pick_splits(uint64_t groups, uint64_t visible) {
    // Enough CTAs to fill 148 SMs a few times over with at least ~256 keys per slice; among those
    // prefer a count that makes groups * splits a whole number of waves (a multiple of the SM count).
    const uint64_t want = ((uint64_t)kSmCount * 4 + groups - 1) / groups;
    const uint64_t cap = (visible + 255) / 256;
    uint64_t s = want < cap ? want : cap;
    s = s < 1 ? 1 : s;
    for (uint64_t t = s; t <= s + 40 && t <= cap && t <= 64; ++t)
        if ((groups * t) % kSmCount == 0) { s = t; break; }
    return (int)(s > 64 ? 64 : s);
}

template <int D, int G>
static int launch_gqa(const uint16_t *q, const uint16_t *k, const uint16_t *v, uint64_t sessions, int kv_heads,
                      uint64_t context, uint64_t visible, float scale, float *out, float *partial, int splits,
                      int *status, cudaStream_t s) {
    static_assert(G <= kMaxGroup, "GQA group does not fit the MMA rows");
    const uint64_t groups = sessions * kv_heads;
    uint64_t per_split = (visible + splits - 1) / splits;
    per_split = (per_split + kKeyBlock - 1) / kKeyBlock * kKeyBlock;       // slices start on 16-key blocks
    gqa_decode_kernel<D><<<(unsigned)(groups * splits), kAttnThreads, 0, s>>>(q, k, v, kv_heads, G, context, visible,
                                                                              scale, splits, per_split, partial, status);
    gqa_merge_kernel<D, G><<<(unsigned)groups, 128, 0, s>>>(partial, splits, groups, out, status);
    return launch_status(2);
}

}  // namespace yb

using namespace yb;

extern "C" uint64_t yvex_b200_attention_workspace_bytes(uint64_t sessions, uint64_t q_heads, uint64_t kv_heads,
                                                        uint64_t head_dim, uint64_t context) {
    if (!kv_heads) return 0;
    int splits = pick_splits(sessions * kv_heads, context);
    return sessions * q_heads * (uint64_t)splits * (head_dim + 2) * sizeof(float);
}

extern "C" int yvex_b200_attention_gqa_decode(const void *q, const void *k, const void *v, uint64_t sessions,
                                              uint64_t q_heads, uint64_t kv_heads, uint64_t head_dim,
                                              uint64_t context, uint64_t position, float scale, float *out,
                                              void *workspace, uint64_t workspace_bytes, int *status, void *stream) {
    if (!q || !k || !v || !out || !status || !sessions || !q_heads || !kv_heads || !context) return ERR_INVALID_ARG;
    if (!isfinite(scale) || scale <= 0.0f) return ERR_INVALID_ARG;            // src/backend/cpu.c:346-350
    if (position >= context) return ERR_BOUNDS;                               // src/backend/core.c:1473-1476
    if (q_heads % kv_heads) return ERR_INVALID_ARG;
    if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v) & 15u) return ERR_INVALID_ARG;
    const uint64_t group = q_heads / kv_heads, visible = position + 1;
    const int splits = pick_splits(sessions * kv_heads, visible);
    const uint64_t need = sessions * q_heads * (uint64_t)splits * (head_dim + 2) * sizeof(float);
    if (!workspace || workspace_bytes < need) return ERR_NOMEM;
    const uint16_t *qq = (const uint16_t *)q, *kk = (const uint16_t *)k, *vv = (const uint16_t *)v;
    float *partial = (float *)workspace;
    cudaStream_t s = as_stream(stream);
#define YB_GQA(DD, GG)                                                                                   \
    if (head_dim == DD && group == GG)                                                                   \
        return launch_gqa<DD, GG>(qq, kk, vv, sessions, (int)kv_heads, context, visible, scale, out, partial, splits, status, s);
    YB_GQA(128, 4) YB_GQA(128, 1) YB_GQA(128, 2) YB_GQA(64, 1) YB_GQA(64, 2) YB_GQA(64, 4)
    YB_GQA(256, 1) YB_GQA(256, 2) YB_GQA(256, 4)
#undef YB_GQA
    return ERR_UNSUPPORTED;
}

extern "C" int yvex_b200_attention_f32(const float *q, const float *keys, const float *values, uint64_t seq_len,
                                       uint64_t head_dim, uint64_t position, float scale, int causal,
                                       float *scores, float *probabilities, float *out, int *status, void *stream) {
    if (!q || !keys || !values || !scores || !probabilities || !out || !status) return ERR_INVALID_ARG;
    if (!isfinite(scale) || scale <= 0.0f) return ERR_INVALID_ARG;
    if (!seq_len || !head_dim) return ERR_FORMAT;
    if (position >= seq_len) return ERR_BOUNDS;
    attention_f32_kernel<<<1, 1024, 0, as_stream(stream)>>>(q, keys, values, seq_len, head_dim,
                                                            causal ? position + 1 : seq_len, scale, scores,
                                                            probabilities, out, status);
    return launch_status();
}

extern "C" int yvex_b200_attention_sink(const float *query, const float *rows, const float *sinks, uint64_t heads, uint64_t row_count,
                                        uint64_t head_dim, double scale, int round_bf16, float *out, int *status, void *stream) {
    if (!query || (!rows && row_count) || !sinks || !out || !status || !heads) return ERR_INVALID_ARG;
    if (!isfinite(scale) || scale <= 0.0) return ERR_INVALID_ARG;
    if (!head_dim || head_dim > 1024) return ERR_BOUNDS;
    attention_sink_kernel<<<(unsigned)heads, 32 * kSinkWarps, 0, as_stream(stream)>>>(query, rows, sinks, row_count, head_dim, scale, round_bf16,
                                                                                      out, status);
    return launch_status();
}
