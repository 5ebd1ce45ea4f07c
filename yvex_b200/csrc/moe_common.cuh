// Types and helpers shared by the MoE kernels (router, narrow/decode path, wide/prefill path).
#pragma once
#include "qtype_decode.cuh"

namespace yb {

using MoeGeom = yvex_b200_moe_geometry;
using MoeWeights = yvex_b200_moe_weights;

// SwiGLU with the reference's clamps and its single bf16 rounding point after the route weight
// (src/graph/moe.c:605-613).
// silu(g) = g / (1 + exp(-g)) for g >= 0 and g * exp(g) / (1 + exp(g)) below: with t = exp(-|g|) both
// are (g or g * t) / (1 + t), the same operations on the same values, evaluated without a branch.
__device__ __forceinline__ float swiglu_product(float g, float u, float route_weight, float limit) {
    g = fminf(g, limit);
    u = fmaxf(-limit, fminf(u, limit));
    const float t = expf(-fabsf(g));
    const float silu = (g >= 0.0f ? g : g * t) / (1.0f + t);
    return silu * u * route_weight;
}
__device__ __forceinline__ float swiglu_mid(float g, float u, float route_weight, float limit, int *status) {
    const float mid = swiglu_product(g, u, route_weight, limit);
    if (!isfinite(mid)) raise(status, YVEX_B200_STATUS_NUMERIC);
    return bf16_round(mid);
}

// Device scratch of the MoE entry points, carved from the caller's workspace in 256-byte
// aligned ranges like the reference's bump allocator (src/backend/cuda/moe.c:78-88).
struct MoeWorkspace {
    float *xr;          // [rows x hidden]  bf16-exact ingress rows
    float *logits;      // [rows x experts]
    float *scores;      // [rows x experts]  sqrt(softplus(logit)) when the router projection ran on device
    int32_t *selected;  // [rows x topk]
    float *weights;     // [rows x topk]
    float *mid;         // [rows x (topk+1) x max(inter, shared_inter)]  SwiGLU intermediates
    __half *xr_h;       // fp16 image of xr (bf16-exact values; B operand of the tensor-core matvecs)
    __half *mid_h;      // fp16 image of mid
    // optional parts of the result, set by the entry point (not scratch): [rows x hidden] f32 each, the
    // rank-ordered sum of the routed experts' rows and the shared expert's row (src/runtime/moe.c:606-637)
    float *routed_out = nullptr, *shared_out = nullptr;
    void rebase(void *base) {
        auto b = reinterpret_cast<uintptr_t>(base);
        xr_h = reinterpret_cast<__half *>(b + reinterpret_cast<uintptr_t>(xr_h));
        mid_h = reinterpret_cast<__half *>(b + reinterpret_cast<uintptr_t>(mid_h));
        xr = reinterpret_cast<float *>(b + reinterpret_cast<uintptr_t>(xr));
        logits = reinterpret_cast<float *>(b + reinterpret_cast<uintptr_t>(logits));
        scores = reinterpret_cast<float *>(b + reinterpret_cast<uintptr_t>(scores));
        selected = reinterpret_cast<int32_t *>(b + reinterpret_cast<uintptr_t>(selected));
        weights = reinterpret_cast<float *>(b + reinterpret_cast<uintptr_t>(weights));
        mid = reinterpret_cast<float *>(b + reinterpret_cast<uintptr_t>(mid));
    }
};

// Fills `ws` with OFFSETS (rebase() turns them into pointers) and returns the total bytes.
inline uint64_t moe_workspace_layout(const MoeGeom &g, uint64_t rows, MoeWorkspace *ws) {
    uint64_t off = 0;
    auto take = [&](uint64_t bytes) { uint64_t at = off; off = (off + bytes + 255) & ~255ull; return at; };
    const uint64_t imax = g.inter > g.shared_inter ? g.inter : g.shared_inter;
    MoeWorkspace l;
    l.xr = reinterpret_cast<float *>(take(rows * g.hidden * 4));
    l.logits = reinterpret_cast<float *>(take(rows * g.experts * 4));
    l.scores = reinterpret_cast<float *>(take(rows * g.experts * 4));
    l.selected = reinterpret_cast<int32_t *>(take(rows * g.topk * 4));
    l.weights = reinterpret_cast<float *>(take(rows * g.topk * 4));
    l.mid = reinterpret_cast<float *>(take(rows * (g.topk + 1) * imax * 4));
    l.xr_h = reinterpret_cast<__half *>(take(rows * g.hidden * 2));
    l.mid_h = reinterpret_cast<__half *>(take(rows * (g.topk + 1) * imax * 2));
    if (ws) *ws = l;
    return off;
}

// Scratch of the streaming decode path, behind the fixed part of the MoE workspace (narrow batches only).
struct DecodeStreamScratch {
    const uint8_t **gu_ptrs, **down_ptrs;      // [pairs * 2], [pairs] matrix addresses
    uint32_t *gu_rows;                         // input row of each gate/up matrix
    float *gu;                                 // [pairs][2][inter]
    float *y;                                  // [pairs][hidden] (bf16-rounded)
    float *pair_weight;                        // [pairs] route weight of the pair (1 for the shared expert)
    void rebase(void *base) {
        auto b = reinterpret_cast<uintptr_t>(base);
        gu_ptrs = reinterpret_cast<const uint8_t **>(b + reinterpret_cast<uintptr_t>(gu_ptrs));
        down_ptrs = reinterpret_cast<const uint8_t **>(b + reinterpret_cast<uintptr_t>(down_ptrs));
        gu_rows = reinterpret_cast<uint32_t *>(b + reinterpret_cast<uintptr_t>(gu_rows));
        gu = reinterpret_cast<float *>(b + reinterpret_cast<uintptr_t>(gu));
        y = reinterpret_cast<float *>(b + reinterpret_cast<uintptr_t>(y));
        pair_weight = reinterpret_cast<float *>(b + reinterpret_cast<uintptr_t>(pair_weight));
    }
};
// What the router's top-k kernel needs to write the streaming decode path's tables itself (one launch less).
struct RouteTables {
    MoeWeights w;
    uint64_t gate_bytes, down_bytes;           // bytes of one expert's gate (= up) and down matrix
    DecodeStreamScratch t;
    int enabled;
};
// pair q = row * (k + 1) + p: p < k the routed expert `expert` with route weight `weight`, p == k the shared expert
__device__ __forceinline__ void write_pair_tables(const RouteTables &rt, uint64_t q, uint32_t row, bool shared, int64_t expert, float weight) {
    rt.t.gu_ptrs[2 * q] = shared ? (const uint8_t *)rt.w.shared_gate : (const uint8_t *)rt.w.gate + (uint64_t)expert * rt.gate_bytes;
    rt.t.gu_ptrs[2 * q + 1] = shared ? (const uint8_t *)rt.w.shared_up : (const uint8_t *)rt.w.up + (uint64_t)expert * rt.gate_bytes;
    rt.t.gu_rows[2 * q] = rt.t.gu_rows[2 * q + 1] = row;
    rt.t.down_ptrs[q] = shared ? (const uint8_t *)rt.w.shared_down : (const uint8_t *)rt.w.down + (uint64_t)expert * rt.down_bytes;
    rt.t.pair_weight[q] = shared ? 1.0f : weight;
}
// Offsets (rebase() turns them into pointers) from `base`; returns the end.
uint64_t moe_decode_stream_layout(const MoeGeom &g, uint64_t rows, uint64_t base, DecodeStreamScratch *out);
bool moe_decode_stream_eligible(const MoeGeom &g, const MoeWeights &w);
// The (k + 1) experts of every row as two batched launches of the streaming matvec (gate/up, down).
int moe_experts_stream(const MoeGeom &g, const MoeWeights &w, const MoeWorkspace &ws, const DecodeStreamScratch &t, bool tables_ready, uint64_t rows,
                       float *out, int *status, cudaStream_t s);

// Expert execution for a narrow batch; picks the streaming tensor-core matvec kernels when the
// layer's qtypes have decoders for them and the reference-shaped kernels otherwise.
int moe_experts_narrow(const MoeGeom &g, const MoeWeights &w, const MoeWorkspace &ws, uint64_t rows,
                       float *out, int *status, cudaStream_t s);
int moe_experts_rows(const MoeGeom &g, const MoeWeights &w, const MoeWorkspace &ws, uint64_t rows,
                     float *out, int *status, cudaStream_t s);
int moe_up_rows(const MoeGeom &g, const MoeWeights &w, const MoeWorkspace &ws, uint64_t rows, int *status,
                cudaStream_t s);
int moe_down_rows(const MoeGeom &g, const MoeWeights &w, const MoeWorkspace &ws, uint64_t rows, float *out,
                  int *status, cudaStream_t s);
// Ingress bf16 rounding of x into ws.xr, then router (projection or supplied logits) + top-k.
int moe_ingress_and_route(const MoeGeom &g, const MoeWeights &w, const MoeWorkspace &ws, const float *x,
                          const float *logits, const uint32_t *token_ids, uint64_t rows, int *status,
                          cudaStream_t s, RouteTables *tables = nullptr);      // tables->enabled is cleared when they were not written
// Entry-point validation shared by the narrow and wide paths (fail-closed qtype check included).
int moe_check_geometry(const yvex_b200_moe_geometry *g, const yvex_b200_moe_weights *w);

}  // namespace yb
