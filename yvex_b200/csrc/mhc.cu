// mHC envelope of the MoE FFN: the layer's input is a row of `streams` residual streams
// (expanded width = streams * hidden); `prepare` collapses it to the FFN input and `post`
// re-expands the FFN output. Arithmetic follows the reference CPU path step by step:
//   mix      = mhc_fn . expanded, double dots                      src/graph/moe.c:458, quant_compute.c:116-181
//   inverse  = 1/sqrt(mean(expanded^2) + rms_eps)                  src/graph/numeric.c:785-792
//   pre[s]   = sigmoid(mix[s]*inverse*scale[0] + base[s])          :794-797
//   post[s]  = mult * sigmoid(mix[S+s]*inverse*scale[1] + base[S+s])   :798-801
//   comb[s][t] = mix[2S+sS+t]*inverse*scale[2] + base[..], then row softmax + eps and
//              `iterations` rounds of row/column normalisation     :802-809, 706-750
//   collapsed = sum_s (float)((pre[s]+eps) * x[s]) in stream order (f32 adds), bf16 round   :810-815
//   normalized = bf16( collapsed * 1/sqrt(mean(collapsed^2)+rms_eps) * norm )   numeric.c:630-659, moe.c:487-489
//   post:  out[t] = bf16( (float)(post[t]*core + sum_s comb[s][t]*x[s]) ), double   numeric.c:855-868
// Launches: one CTA per (mix row, token row) for the dots (plus one per token row for the sum of
// squares), one CTA per token row for gates + Sinkhorn + collapse + RMSNorm, an elementwise kernel
// for post.
#include "common.cuh"

namespace yb {

constexpr int kMhcThreads = 128;
constexpr int kMhcRowThreads = 1024;
constexpr int kMhcMaxStreams = 6;            // (streams + 2) * streams <= 64 mixing rows (src/graph/moe.c:455)
constexpr int kMhcMaxPerThread = 16;         // hidden <= 16384 (src/graph/moe.c:456)

__device__ __forceinline__ double block_sum(double v, double *scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();                                     // scratch may still be read from a previous call
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    double total = 0.0;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) total += scratch[i];
    return total;
}

// blockIdx.x < mix_rows: mix[row][blockIdx.x]; blockIdx.x == mix_rows: squares[row].
__global__ void __launch_bounds__(kMhcThreads)
mhc_mix_kernel(const float *fn, const float *expanded, uint64_t width, int mix_rows, float *mix, double *squares, int *status) {
    __shared__ double scratch[kMhcThreads / 32];
    const uint64_t r = blockIdx.y;
    const float *x = expanded + r * width;
    const bool dot = (int)blockIdx.x < mix_rows;
    const float *w = dot ? fn + (uint64_t)blockIdx.x * width : x;
    double acc = 0.0;
    bool bad = false;
    const uint64_t vec = width / 4;
    for (uint64_t base = 0; base < vec; base += 4 * kMhcThreads) {
        float4 wv[4], xv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint64_t at = base + (uint64_t)i * kMhcThreads + threadIdx.x;
            const bool in = at < vec;
            xv[i] = in ? __ldg(reinterpret_cast<const float4 *>(x) + at) : make_float4(0.f, 0.f, 0.f, 0.f);
            wv[i] = dot ? (in ? __ldg(reinterpret_cast<const float4 *>(w) + at) : make_float4(0.f, 0.f, 0.f, 0.f)) : xv[i];
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            bad |= !isfinite(xv[i].x) || !isfinite(xv[i].y) || !isfinite(xv[i].z) || !isfinite(xv[i].w);
            acc += (double)wv[i].x * (double)xv[i].x;
            acc += (double)wv[i].y * (double)xv[i].y;
            acc += (double)wv[i].z * (double)xv[i].z;
            acc += (double)wv[i].w * (double)xv[i].w;
        }
    }
    const double total = block_sum(acc, scratch);
    if (bad) raise(status, YVEX_B200_STATUS_NUMERIC);
    if (threadIdx.x == 0) {
        if (dot) {
            const float v = (float)total;
            if (!isfinite(v)) raise(status, YVEX_B200_STATUS_NUMERIC);
            mix[r * mix_rows + blockIdx.x] = v;
        } else {
            squares[r] = total;
        }
    }
}

__device__ __forceinline__ double sigmoid_d(double v) {
    if (v >= 0.0) return 1.0 / (1.0 + exp(-v));
    const double d = exp(v);
    return d / (1.0 + d);
}

// One CTA per token row.
__global__ void __launch_bounds__(kMhcRowThreads)
mhc_collapse_kernel(yvex_b200_mhc m, const float *expanded, const float *mix, const double *squares, float *normalized,
                    float *post, float *combination, int *status) {
    __shared__ double scratch[kMhcRowThreads / 32];
    __shared__ double pre[kMhcMaxStreams];
    __shared__ int failed;
    const uint64_t r = blockIdx.x, H = m.hidden, S = m.streams, W = S * H;
    const int rows = (int)((S + 2) * S);
    const float *x = expanded + r * W;
    if (threadIdx.x == 0) {
        failed = 0;
        const float *mx = mix + r * rows;
        const double inv = 1.0 / sqrt(squares[r] / (double)W + m.rms_epsilon);
        bool ok = isfinite(inv);
        for (int i = 0; i < 3; ++i) ok &= isfinite(m.scale[i]);
        for (int i = 0; i < rows; ++i) ok &= isfinite(m.base[i]);
        float c[kMhcMaxStreams * kMhcMaxStreams];
        for (uint64_t s = 0; s < S; ++s) {
            pre[s] = sigmoid_d((double)mx[s] * inv * (double)m.scale[0] + (double)m.base[s]);
            post[r * S + s] = (float)(m.post_multiplier * sigmoid_d((double)mx[S + s] * inv * (double)m.scale[1] + (double)m.base[S + s]));
            for (uint64_t t = 0; t < S; ++t) {
                const uint64_t idx = 2 * S + s * S + t;
                c[s * S + t] = (float)((double)mx[idx] * inv * (double)m.scale[2] + (double)m.base[idx]);
            }
        }
        // Sinkhorn normalisation of the stream combination (src/graph/numeric.c:706-750)
        for (uint64_t row = 0; row < S && ok; ++row) {
            double mxv = -(double)INFINITY, total = 0.0;
            for (uint64_t col = 0; col < S; ++col) mxv = fmax(mxv, (double)c[row * S + col]);
            for (uint64_t col = 0; col < S; ++col) {
                const double v = exp((double)c[row * S + col] - mxv);
                c[row * S + col] = (float)v;
                total += v;
            }
            ok &= isfinite(total) && total > 0.0;
            for (uint64_t col = 0; col < S; ++col) c[row * S + col] = (float)((double)c[row * S + col] / total + m.mhc_epsilon);
        }
        for (uint64_t it = 0; it < m.sinkhorn_iterations && ok; ++it) {
            if (it != 0) {
                for (uint64_t row = 0; row < S; ++row) {
                    double total = 0.0;
                    for (uint64_t col = 0; col < S; ++col) total += c[row * S + col];
                    ok &= isfinite(total);
                    for (uint64_t col = 0; col < S; ++col) c[row * S + col] = (float)((double)c[row * S + col] / (total + m.mhc_epsilon));
                }
            }
            for (uint64_t col = 0; col < S; ++col) {
                double total = 0.0;
                for (uint64_t row = 0; row < S; ++row) total += c[row * S + col];
                ok &= isfinite(total);
                for (uint64_t row = 0; row < S; ++row) c[row * S + col] = (float)((double)c[row * S + col] / (total + m.mhc_epsilon));
            }
        }
        for (uint64_t i = 0; i < S * S; ++i) combination[r * S * S + i] = c[i];
        if (!ok) failed = 1;
    }
    __syncthreads();
    if (failed) { if (threadIdx.x == 0) raise(status, YVEX_B200_STATUS_NUMERIC); return; }
    float v[kMhcMaxPerThread];
    double sq = 0.0;
    bool bad = false;
#pragma unroll
    for (int j = 0; j < kMhcMaxPerThread; ++j) {
        const uint64_t i = (uint64_t)j * kMhcRowThreads + threadIdx.x;
        v[j] = 0.0f;
        if (i < H) {
            float acc = 0.0f;
            for (uint64_t s = 0; s < S; ++s) acc += (float)((pre[s] + m.mhc_epsilon) * (double)x[s * H + i]);
            bad |= !isfinite(acc) || !isfinite(m.norm[i]);
            acc = bf16_round(acc);
            v[j] = acc;
            sq += (double)acc * (double)acc;
        }
    }
    const double mean = block_sum(sq, scratch) / (double)H;
    const double ninv = 1.0 / sqrt(mean + m.rms_epsilon);
    if (bad || !isfinite(ninv)) { raise(status, YVEX_B200_STATUS_NUMERIC); return; }
#pragma unroll
    for (int j = 0; j < kMhcMaxPerThread; ++j) {
        const uint64_t i = (uint64_t)j * kMhcRowThreads + threadIdx.x;
        if (i < H) {
            const double o = (double)v[j] * ninv * (double)m.norm[i];
            if (!isfinite(o)) raise(status, YVEX_B200_STATUS_NUMERIC);
            normalized[r * H + i] = bf16_round((float)o);
        }
    }
}

__global__ void mhc_post_kernel(const float *core, const float *expanded, const float *post, const float *combination,
                                uint64_t streams, uint64_t hidden, uint64_t rows, float *out, int *status) {
    const uint64_t W = streams * hidden, total = rows * W;
    for (uint64_t idx = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; idx < total; idx += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t r = idx / W, local = idx % W, t = local / hidden, i = local % hidden;
        double v = (double)post[r * streams + t] * (double)core[r * hidden + i];
        for (uint64_t s = 0; s < streams; ++s)
            v += (double)combination[(r * streams + s) * streams + t] * (double)expanded[r * W + s * hidden + i];
        const float o = (float)v;
        if (!isfinite(o)) raise(status, YVEX_B200_STATUS_NUMERIC);
        out[idx] = bf16_round(o);
    }
}

static int check_mhc(const yvex_b200_mhc *m) {
    if (!m || !m->mhc_fn || !m->scale || !m->base || !m->norm) return ERR_INVALID_ARG;
    if (!m->hidden || !m->streams || !m->sinkhorn_iterations) return ERR_INVALID_ARG;
    if (m->streams > (uint64_t)kMhcMaxStreams || m->hidden > (uint64_t)kMhcMaxPerThread * kMhcRowThreads) return ERR_BOUNDS;
    if (m->hidden % 4) return ERR_BOUNDS;
    if (!(m->rms_epsilon > 0.0) || !(m->mhc_epsilon > 0.0) || !(m->post_multiplier > 0.0) || !isfinite(m->rms_epsilon) ||
        !isfinite(m->mhc_epsilon) || !isfinite(m->post_multiplier))
        return ERR_INVALID_ARG;                                           // src/graph/numeric.c:688-692
    return OK;
}

}  // namespace yb

using namespace yb;

extern "C" uint64_t yvex_b200_mhc_workspace_bytes(uint64_t streams, uint64_t rows) {
    const uint64_t mix = (rows * (streams + 2) * streams * sizeof(float) + 255) & ~255ull;
    return mix + ((rows * sizeof(double) + 255) & ~255ull);
}

extern "C" int yvex_b200_mhc_prepare(const yvex_b200_mhc *m, const float *expanded, uint64_t rows, float *normalized,
                                     float *post, float *combination, void *workspace, uint64_t workspace_bytes,
                                     int *status, void *stream) {
    int rc = check_mhc(m);
    if (rc != OK) return rc;
    if (!expanded || !normalized || !post || !combination || !status || !rows || rows > 65535) return ERR_INVALID_ARG;
    if ((reinterpret_cast<uintptr_t>(expanded) | reinterpret_cast<uintptr_t>(m->mhc_fn)) & 15u) return ERR_INVALID_ARG;
    if (!workspace || workspace_bytes < yvex_b200_mhc_workspace_bytes(m->streams, rows)) return ERR_NOMEM;
    const int mix_rows = (int)((m->streams + 2) * m->streams);
    float *mix = static_cast<float *>(workspace);
    double *squares = reinterpret_cast<double *>(static_cast<uint8_t *>(workspace) +
                                                 ((rows * mix_rows * sizeof(float) + 255) & ~255ull));
    cudaStream_t s = as_stream(stream);
    mhc_mix_kernel<<<dim3((unsigned)mix_rows + 1u, (unsigned)rows), kMhcThreads, 0, s>>>(
        m->mhc_fn, expanded, m->streams * m->hidden, mix_rows, mix, squares, status);
    mhc_collapse_kernel<<<(unsigned)rows, kMhcRowThreads, 0, s>>>(*m, expanded, mix, squares, normalized, post, combination, status);
    return launch_status(2);
}

extern "C" int yvex_b200_mhc_post(const yvex_b200_mhc *m, const float *core, const float *expanded, const float *post,
                                  const float *combination, uint64_t rows, float *out, int *status, void *stream) {
    int rc = check_mhc(m);
    if (rc != OK) return rc;
    if (!core || !expanded || !post || !combination || !out || !status || !rows) return ERR_INVALID_ARG;
    const uint64_t total = rows * m->streams * m->hidden;
    mhc_post_kernel<<<grid_for(total, 256, 8), 256, 0, as_stream(stream)>>>(core, expanded, post, combination, m->streams,
                                                                           m->hidden, rows, out, status);
    return launch_status(1);
}
