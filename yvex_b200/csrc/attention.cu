// Online-softmax attention.
//
// gqa_decode: one query position per session against a bf16 KV cache. The cache is the only
// traffic that matters (2 x context x head_dim x 2 bytes per KV head), so the kernel is built to
// stream it once: a CTA owns one (session, KV head) and one slice of the context, all q heads of
// the GQA group share every K/V load, D/8 lanes read one 16-byte chunk each of a key row
// (fully coalesced 128-bit loads), scores are kept in f32 and the running (max, sum, accumulator)
// triple is rescaled once per 8-key block. Slices are merged by a second tiny kernel
// (log-sum-exp merge). Math per (session, q head) is the reference CPU op's: scores =
// scale * q.k, softmax over keys 0..position, out = sum p*v (src/backend/cpu.c:319-411).
#include "common.cuh"

namespace yb {

constexpr int kAttnThreads = 256;
constexpr int kKeyBlock = 8;

__device__ __forceinline__ void bf16x8_to_float(const uint4 &raw, float (&f)[8]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

// Partial layout per (session, kv head, split): G heads x (m, l, acc[D]).
template <int D, int G>
__global__ void __launch_bounds__(kAttnThreads)
gqa_decode_kernel(const uint16_t *__restrict__ q, const uint16_t *__restrict__ k,
                  const uint16_t *__restrict__ v, int kv_heads, uint64_t context, uint64_t visible,
                  float scale, int splits, float *__restrict__ partial, int *status) {
    constexpr int LPK = D / 8;                 // lanes per key row
    constexpr int KPW = 32 / LPK;              // keys a warp reads per load instruction
    constexpr int NW = kAttnThreads / 32;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane / LPK, ll = lane % LPK;     // key slot inside the warp, chunk inside the row
    // Key slots of one warp may run different trip counts at the ragged end of a split, so the
    // score reduction synchronises only the lanes of its own slot.
    const unsigned slot_mask = static_cast<unsigned>(((1ull << LPK) - 1ull) << (sub * LPK));
    const int split = blockIdx.x % splits;
    const uint64_t sk = blockIdx.x / splits;           // session * kv_heads + kv head
    const uint64_t session = sk / kv_heads, kvh = sk % kv_heads;
    const uint16_t *kb = k + sk * context * D, *vb = v + sk * context * D;
    const uint16_t *qb = q + (session * (uint64_t)kv_heads * G + kvh * G) * D;

    float qf[G][8];
#pragma unroll
    for (int h = 0; h < G; ++h) {
        uint4 raw = __ldg(reinterpret_cast<const uint4 *>(qb + h * D) + ll);
        bf16x8_to_float(raw, qf[h]);
#pragma unroll
        for (int i = 0; i < 8; ++i) qf[h][i] *= scale;
    }
    float m[G], l[G], acc[G][8];
#pragma unroll
    for (int h = 0; h < G; ++h) {
        m[h] = -INFINITY; l[h] = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[h][i] = 0.0f;
    }
    // This split's key range, in units of kKeyBlock*KPW*NW keys so every slot stays balanced.
    const uint64_t per_split = (visible + splits - 1) / splits;
    const uint64_t begin = (uint64_t)split * per_split;
    const uint64_t end = begin + per_split < visible ? begin + per_split : visible;
    const uint64_t stride = (uint64_t)NW * KPW * kKeyBlock;
    for (uint64_t base = begin + ((uint64_t)warp * KPW + sub) * kKeyBlock; base < end; base += stride) {
        float s[kKeyBlock][G];
        uint4 kraw[kKeyBlock];
#pragma unroll
        for (int j = 0; j < kKeyBlock; ++j) {
            const uint64_t key = base + j;
            kraw[j] = key < end ? __ldg(reinterpret_cast<const uint4 *>(kb + key * D) + ll) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int j = 0; j < kKeyBlock; ++j) {
            float kf[8];
            bf16x8_to_float(kraw[j], kf);
#pragma unroll
            for (int h = 0; h < G; ++h) {
                float d = 0.0f;
#pragma unroll
                for (int i = 0; i < 8; ++i) d = fmaf(qf[h][i], kf[i], d);
#pragma unroll
                for (int o = LPK / 2; o > 0; o >>= 1) d += __shfl_xor_sync(slot_mask, d, o);
                s[j][h] = base + j < end ? d : -INFINITY;
            }
        }
        uint4 vraw[kKeyBlock];
#pragma unroll
        for (int j = 0; j < kKeyBlock; ++j) {
            const uint64_t key = base + j;
            vraw[j] = key < end ? __ldg(reinterpret_cast<const uint4 *>(vb + key * D) + ll) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int h = 0; h < G; ++h) {
            float bm = m[h];
#pragma unroll
            for (int j = 0; j < kKeyBlock; ++j) bm = fmaxf(bm, s[j][h]);
            const float corr = __expf(m[h] - bm);     // m = -inf on the first block -> 0
            m[h] = bm;
            l[h] *= corr;
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[h][i] *= corr;
#pragma unroll
            for (int j = 0; j < kKeyBlock; ++j) s[j][h] = __expf(s[j][h] - bm);
        }
#pragma unroll
        for (int j = 0; j < kKeyBlock; ++j) {
            float vf[8];
            bf16x8_to_float(vraw[j], vf);
#pragma unroll
            for (int h = 0; h < G; ++h) {
                l[h] += s[j][h];
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[h][i] = fmaf(s[j][h], vf[i], acc[h][i]);
            }
        }
    }
    // Merge the NW*KPW key slots of the CTA through shared memory.
    __shared__ float sm_m[NW * KPW][G], sm_l[NW * KPW][G];
    __shared__ float sm_acc[NW * KPW][G][D];
    const int slot = warp * KPW + sub;
#pragma unroll
    for (int h = 0; h < G; ++h) {
        if (ll == 0) { sm_m[slot][h] = m[h]; sm_l[slot][h] = l[h]; }
#pragma unroll
        for (int i = 0; i < 8; ++i) sm_acc[slot][h][ll * 8 + i] = acc[h][i];
    }
    __syncthreads();
    float *po = partial + ((sk * splits + split) * G) * (uint64_t)(D + 2);
    for (int idx = threadIdx.x; idx < G * D; idx += kAttnThreads) {
        const int h = idx / D, d = idx % D;
        float gm = -INFINITY;
        for (int sidx = 0; sidx < NW * KPW; ++sidx) gm = fmaxf(gm, sm_m[sidx][h]);
        float gl = 0.0f, ga = 0.0f;
        for (int sidx = 0; sidx < NW * KPW; ++sidx) {
            const float c = sm_m[sidx][h] == -INFINITY ? 0.0f : __expf(sm_m[sidx][h] - gm);
            gl += sm_l[sidx][h] * c;
            ga += sm_acc[sidx][h][d] * c;
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

static int pick_splits(uint64_t groups, uint64_t visible) {
    // enough CTAs to fill 148 SMs a few times over, but at least ~512 keys per split
    uint64_t want = ((uint64_t)kSmCount * 4 + groups - 1) / groups;
    uint64_t cap = (visible + 511) / 512;
    uint64_t s = want < cap ? want : cap;
    return (int)(s < 1 ? 1 : s > 64 ? 64 : s);
}

template <int D, int G>
static int launch_gqa(const uint16_t *q, const uint16_t *k, const uint16_t *v, uint64_t sessions, int kv_heads,
                      uint64_t context, uint64_t visible, float scale, float *out, float *partial, int splits,
                      int *status, cudaStream_t s) {
    const uint64_t groups = sessions * kv_heads;
    gqa_decode_kernel<D, G><<<(unsigned)(groups * splits), kAttnThreads, 0, s>>>(q, k, v, kv_heads, context, visible,
                                                                                   scale, splits, partial, status);
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
