// Elementwise steps of the token-local MoE transaction (begin / add_expert / finish of the host
// boundary), which runs one expert at a time like the reference's
// yvex_backend_moe_add_expert (src/backend/cuda/moe.c:673-724): the matvecs are yvex_b200_gemv, these
// are what sits between them. Each kernel is the device twin of one loop of the CPU layer
// (src/graph/moe.c:487-489, :497-519, :587-622; src/runtime/moe.c:620-632).
#include "moe_common.cuh"

namespace yb {

// ingress: the normalized row is bf16-exact (src/graph/moe.c:487-489)
__global__ void token_round_kernel(const float *x, uint64_t n, float *out, int *status) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const float v = x[i];
        if (!isfinite(v)) raise(status, YVEX_B200_STATUS_NUMERIC);
        out[i] = bf16_round(v);
    }
}

// score = (float)sqrt(softplus(logit)), in double (src/graph/moe.c:497-506)
__global__ void token_scores_kernel(const float *logits, uint64_t n, float *scores, int *status) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const double v = logits[i];
        const double sp = v > 0.0 ? v + log1p(exp(-v)) : log1p(exp(v));
        const double s = sqrt(sp);
        if (!isfinite(s)) raise(status, YVEX_B200_STATUS_NUMERIC);
        scores[i] = (float)s;
    }
}

// mid = bf16(silu(min(g, limit)) * clamp(u, +-limit) * weight) (src/graph/moe.c:604-616)
__global__ void token_swiglu_kernel(const float *gate, const float *up, uint64_t n, float limit, float weight, float *mid, int *status) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
        mid[i] = swiglu_mid(gate[i], up[i], weight, limit, status);
}

// dst += src in f32, one expert after another in the caller's order (src/runtime/moe.c:620-622)
__global__ void token_accumulate_kernel(const float *src, uint64_t n, float *dst, int *status) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const float v = dst[i] + src[i];
        if (!isfinite(v)) raise(status, YVEX_B200_STATUS_NUMERIC);
        dst[i] = v;
    }
}

// out = bf16(a + b) (src/runtime/moe.c:630-634)
__global__ void token_sum_round_kernel(const float *a, const float *b, uint64_t n, float *out, int *status) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const float v = a[i] + b[i];
        if (!isfinite(v)) raise(status, YVEX_B200_STATUS_NUMERIC);
        out[i] = bf16_round(v);
    }
}

}  // namespace yb

using namespace yb;

extern "C" int yvex_b200_moe_token_round(const float *x, uint64_t n, float *out, int *status, void *stream) {
    if (!x || !out || !status || !n) return ERR_INVALID_ARG;
    token_round_kernel<<<grid_for(n, 256, 4), 256, 0, as_stream(stream)>>>(x, n, out, status);
    return launch_status();
}

extern "C" int yvex_b200_moe_token_scores(const float *logits, uint64_t n, float *scores, int *status, void *stream) {
    if (!logits || !scores || !status || !n) return ERR_INVALID_ARG;
    token_scores_kernel<<<grid_for(n, 256, 1), 256, 0, as_stream(stream)>>>(logits, n, scores, status);
    return launch_status();
}

extern "C" int yvex_b200_moe_token_swiglu(const float *gate, const float *up, uint64_t n, double limit, float weight, float *mid,
                                          int *status, void *stream) {
    if (!gate || !up || !mid || !status || !n) return ERR_INVALID_ARG;
    if (!(limit > 0.0) || !isfinite(weight)) return ERR_INVALID_ARG;
    token_swiglu_kernel<<<grid_for(n, 256, 4), 256, 0, as_stream(stream)>>>(gate, up, n, (float)limit, weight, mid, status);
    return launch_status();
}

extern "C" int yvex_b200_moe_token_accumulate(const float *src, uint64_t n, float *dst, int *status, void *stream) {
    if (!src || !dst || !status || !n) return ERR_INVALID_ARG;
    token_accumulate_kernel<<<grid_for(n, 256, 4), 256, 0, as_stream(stream)>>>(src, n, dst, status);
    return launch_status();
}

extern "C" int yvex_b200_moe_token_sum_round(const float *a, const float *b, uint64_t n, float *out, int *status, void *stream) {
    if (!a || !b || !out || !status || !n) return ERR_INVALID_ARG;
    token_sum_round_kernel<<<grid_for(n, 256, 4), 256, 0, as_stream(stream)>>>(a, b, n, out, status);
    return launch_status();
}
