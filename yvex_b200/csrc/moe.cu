// MoE FFN layer: ingress rounding, router scoring + top-k, expert matvecs with the SwiGLU epilogue,
// rank-ordered combine. Numerics follow the reference CPU path step by step:
//   ingress  bf16(x)                               src/graph/moe.c:487-489
//   router   logits (double dot) -> sqrt(softplus) -> biased top-k, lowest index wins ties ->
//            unbiased scores normalised over the selection * scaling     src/graph/moe.c:497-585
//   expert   g=min(gate.x,L) u=clamp(up.x,+-L) mid=bf16(silu(g)*u*w) y=bf16(down.mid)   :587-622
//   combine  routed = sum over ranks in rank order (f32), out = bf16(routed + shared)
//                                                                src/runtime/moe.c:607-632
#include "moe_common.cuh"

namespace yb {

// ---- ingress: x -> bf16-exact f32 rows ----------------------------------------------------------
__global__ void ingress_round_kernel(const float *x, float *xr, __half *xr_h, uint64_t n, int *status) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n;
         i += (uint64_t)gridDim.x * blockDim.x) {
        float v = x[i];
        if (!isfinite(v)) raise(status, YVEX_B200_STATUS_NUMERIC);
        v = bf16_round(v);
        xr[i] = v;
        xr_h[i] = __float2half_rn(v);      // exact for |v| in [2^-14, 65504]; below that < 2^-25 absolute
    }
}

// ---- router projection: one warp per (row, expert), double accumulation -------------------------
__global__ void router_logits_kernel(const float *router, const float *xr, uint64_t rows,
                                     uint64_t experts, uint64_t hidden, float *logits, int *status) {
    const int lane = threadIdx.x & 31;
    const uint64_t warps = (uint64_t)gridDim.x * (blockDim.x >> 5);
    for (uint64_t job = blockIdx.x * (uint64_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
         job < rows * experts; job += warps) {
        const float *w = router + (job % experts) * hidden, *x = xr + (job / experts) * hidden;
        double acc = 0.0;
        for (uint64_t c = lane; c < hidden; c += 32) acc += (double)__ldg(w + c) * (double)__ldg(x + c);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) {
            float v = (float)acc;
            if (!isfinite(v)) raise(status, YVEX_B200_STATUS_NUMERIC);
            logits[job] = v;
        }
    }
}

// ---- decode-width router: ingress rounding + projection + score in one launch ---------------------
// One CTA per (expert, row): dot of the expert's router row with the bf16-rounded input in double
// (same arithmetic as router_logits_kernel), then score = sqrt(softplus(logit)) in double
// (src/graph/moe.c:497-512) so that the top-k kernel only compares. Every CTA also writes its
// interleaved share of the rounded row (f32 and its fp16 image) for the expert kernels.
constexpr int kRouterThreads = 128;
__global__ void __launch_bounds__(kRouterThreads)
ingress_router_kernel(const float *router, const float *x, uint64_t experts, uint64_t hidden, float *xr, __half *xr_h,
                      float *logits, float *scores, int *status) {
    const uint64_t e = blockIdx.x, r = blockIdx.y;
    const float *w = router + e * hidden, *xrow = x + r * hidden;
    pdl_wait();                                         // x may be the output of the kernel before
    pdl_trigger();
    bool bad = false;
    for (uint64_t k = e * kRouterThreads + threadIdx.x; k < hidden; k += experts * kRouterThreads) {
        float v = xrow[k];
        bad |= !isfinite(v);
        v = bf16_round(v);
        xr[r * hidden + k] = v;
        xr_h[r * hidden + k] = __float2half_rn(v);
    }
    double acc = 0.0;
    const uint64_t vec = hidden / 4;            // float4 groups (hidden is a multiple of the block width)
    for (uint64_t base = 0; base < vec; base += 4 * kRouterThreads) {
        float4 wv[4], xv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint64_t at = base + (uint64_t)i * kRouterThreads + threadIdx.x;
            const bool in = at < vec;
            wv[i] = in ? __ldg(reinterpret_cast<const float4 *>(w) + at) : make_float4(0.f, 0.f, 0.f, 0.f);
            xv[i] = in ? __ldg(reinterpret_cast<const float4 *>(xrow) + at) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            acc += (double)wv[i].x * (double)bf16_round(xv[i].x);
            acc += (double)wv[i].y * (double)bf16_round(xv[i].y);
            acc += (double)wv[i].z * (double)bf16_round(xv[i].z);
            acc += (double)wv[i].w * (double)bf16_round(xv[i].w);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    __shared__ double part[kRouterThreads / 32];
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
    if (bad) raise(status, YVEX_B200_STATUS_NUMERIC);
    __syncthreads();
    if (threadIdx.x == 0) {
        double total = 0.0;
        for (int i = 0; i < kRouterThreads / 32; ++i) total += part[i];
        const float logit = (float)total;
        const double v = logit;
        const double sp = v > 0.0 ? v + log1p(exp(-v)) : log1p(exp(v));
        const double sc = sqrt(sp);
        if (!isfinite(logit) || !isfinite(sc)) raise(status, YVEX_B200_STATUS_NUMERIC);
        logits[r * experts + e] = logit;
        scores[r * experts + e] = (float)sc;
    }
}

// ---- scoring + top-k: one warp per row, experts <= 256 (8 per lane), topk <= 16 ------------------
__global__ void route_rows_kernel(MoeGeom g, const float *logits, const float *scores_in, const float *bias,
                                  const int32_t *hash_table, const uint32_t *token_ids,
                                  uint64_t rows, int32_t *selected, float *weights, int *status, const RouteTables rt) {
    const int lane = threadIdx.x & 31;
    const uint64_t row = blockIdx.x * (uint64_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
    pdl_wait();                                         // logits / scores come from the kernel before
    pdl_trigger();
    if (row >= rows) return;
    float score[8], biased[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint64_t e = lane + 32u * i;
        score[i] = 0.0f;
        biased[i] = -INFINITY;
        if (e < g.experts) {
            if (scores_in) {
                score[i] = scores_in[row * g.experts + e];
            } else {
                double v = logits[row * g.experts + e];
                double sp = v > 0.0 ? v + log1p(exp(-v)) : log1p(exp(v));
                double s = sqrt(sp);
                if (!isfinite(s)) raise(status, YVEX_B200_STATUS_NUMERIC);
                score[i] = (float)s;
            }
            biased[i] = (bias ? bias[e] : 0.0f) + score[i];
        }
    }
    int32_t mine = -1;       // lane r keeps the expert selected at rank r
    float mine_w = 0.0f;
    if (g.router_class == 0) {
        bool ok = token_ids && hash_table && token_ids[row] < g.hash_rows;
        if (!ok) { raise(status, YVEX_B200_STATUS_ARGUMENT); return; }
        const int32_t *tr = hash_table + (g.hash_stored_rows == 1 ? 0 : (uint64_t)token_ids[row] * g.topk);
        if ((uint64_t)lane < g.topk) {
            mine = tr[lane];
            if (mine < 0 || (uint64_t)mine >= g.experts) { raise(status, YVEX_B200_STATUS_ARGUMENT); mine = 0; }
        }
        // duplicate selection is an error in the reference (src/graph/moe.c:566-570)
        for (uint64_t r = 0; r < g.topk; ++r) {
            int32_t other = __shfl_sync(0xffffffffu, mine, (int)r);
            if ((uint64_t)lane < g.topk && (uint64_t)lane > r && other == mine) raise(status, YVEX_B200_STATUS_ARGUMENT);
        }
    } else {
        // k rounds of arg-max over the biased scores, lowest index winning ties (src/graph/moe.c:541-556). A float's bit pattern
        // becomes an unsigned key of the same order (sign bit flipped for positives, all bits for negatives; -0 was made +0), so
        // one warp reduction finds the largest value and a second the lowest expert that holds it; a key of 0 stands for
        // "consumed or not an expert". The winning lane hands the expert's unbiased score over in the same round.
        const int topk = (int)g.topk, experts = (int)g.experts;
        uint32_t key[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t bits = __float_as_uint(biased[i] + 0.0f);
            key[i] = lane + 32 * i < experts && biased[i] == biased[i] ? bits ^ ((bits >> 31) ? 0xffffffffu : 0x80000000u) : 0u;      // a NaN is never chosen
        }
        for (int r = 0; r < topk; ++r) {
            uint32_t best = 0u;
            int best_e = 0x7fffffff;
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (key[i] > best) { best = key[i]; best_e = lane + 32 * i; }        // ascending e within a lane: the first maximum stays
            const uint32_t top = __reduce_max_sync(0xffffffffu, best);
            if (top == 0u) { raise(status, YVEX_B200_STATUS_NUMERIC); break; }
            const int win = (int)__reduce_min_sync(0xffffffffu, (unsigned)(best == top ? best_e : 0x7fffffff));
            float s = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) if (win == lane + 32 * i) { s = score[i]; key[i] = 0u; }
            s = __shfl_sync(0xffffffffu, s, win & 31);
            if (lane == r) { mine = win; mine_w = s; }
        }
    }
    if (g.router_class == 0) {
        // weight of rank r = unbiased score of its expert
        for (uint64_t r = 0; r < g.topk; ++r) {
            int32_t e = __shfl_sync(0xffffffffu, mine, (int)r);
            float s = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) if (e == lane + 32 * i) s = score[i];
            s = __shfl_sync(0xffffffffu, s, e & 31);
            if ((uint64_t)lane == r) mine_w = s;
        }
    }
    double total = 0.0;
    for (uint64_t r = 0; r < g.topk; ++r) total += (double)__shfl_sync(0xffffffffu, mine_w, (int)r);
    if (g.normalize && (!isfinite(total) || total <= 0.0)) raise(status, YVEX_B200_STATUS_NUMERIC);
    if ((uint64_t)lane < g.topk) {
        double v = mine_w;
        if (g.normalize) v /= total;
        v *= g.scaling;
        selected[row * g.topk + lane] = mine;
        weights[row * g.topk + lane] = (float)v;
        if (rt.enabled) write_pair_tables(rt, row * (g.topk + 1) + lane, (uint32_t)row, false, mine, (float)v);
    } else if (rt.enabled && (uint64_t)lane == g.topk) {
        write_pair_tables(rt, row * (g.topk + 1) + lane, (uint32_t)row, true, 0, 1.0f);
    }
}

// ---- reference-shaped expert kernels (any supported qtype): one warp per output element ---------
// pair p of row r: p < topk -> routed expert selected[r][p] with weights[r][p]; p == topk -> shared.
__global__ void expert_up_rows_kernel(MoeGeom g, MoeWeights w, const float *xr, const int32_t *selected,
                                      const float *weights, uint64_t rows, float *mid, __half *mid_h,
                                      int *status) {
    const int lane = threadIdx.x & 31;
    const uint64_t ppr = g.topk + 1, imax = max(g.inter, g.shared_inter);
    const uint64_t warps = (uint64_t)gridDim.x * (blockDim.x >> 5);
    const Geometry gg = geometry_of(g.gate_qtype), ug = geometry_of(g.up_qtype);
    const uint64_t grb = g.hidden / gg.elems * gg.bytes, urb = g.hidden / ug.elems * ug.bytes;
    for (uint64_t job = blockIdx.x * (uint64_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
         job < rows * ppr * imax; job += warps) {
        const uint64_t i = job % imax, pair = job / imax, r = pair / ppr, p = pair % ppr;
        const bool shared = p == g.topk;
        const uint64_t width = shared ? g.shared_inter : g.inter;
        if (i >= width) continue;
        const uint8_t *gate, *up;
        float rw = 1.0f;
        if (shared) {
            gate = (const uint8_t *)w.shared_gate + i * grb;
            up = (const uint8_t *)w.shared_up + i * urb;
        } else {
            const uint64_t e = (uint64_t)selected[r * g.topk + p];
            gate = (const uint8_t *)w.gate + (e * g.inter + i) * grb;
            up = (const uint8_t *)w.up + (e * g.inter + i) * urb;
            rw = weights[r * g.topk + p];
        }
        const float *x = xr + r * g.hidden;
        float ga = 0.0f, ua = 0.0f;
        for (uint64_t c = lane; c < g.hidden; c += 32) {
            const float xv = __ldg(x + c);
            ga = fmaf(decode_element(g.gate_qtype, gate + (c / gg.elems) * gg.bytes, (unsigned)(c % gg.elems), status), xv, ga);
            ua = fmaf(decode_element(g.up_qtype, up + (c / ug.elems) * ug.bytes, (unsigned)(c % ug.elems), status), xv, ua);
        }
        ga = warp_sum(ga);
        ua = warp_sum(ua);
        if (lane == 0) {
            const float v = swiglu_mid(ga, ua, rw, (float)g.limit, status);
            mid[pair * imax + i] = v;
            mid_h[pair * imax + i] = __float2half_rn(v);
        }
    }
}

__global__ void expert_down_rows_kernel(MoeGeom g, MoeWeights w, const int32_t *selected, const float *mid,
                                        uint64_t rows, float *out, float *routed_out, float *shared_out, int *status) {
    const int lane = threadIdx.x & 31;
    const uint64_t ppr = g.topk + 1, imax = max(g.inter, g.shared_inter);
    const uint64_t warps = (uint64_t)gridDim.x * (blockDim.x >> 5);
    const Geometry dg = geometry_of(g.down_qtype);
    for (uint64_t job = blockIdx.x * (uint64_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
         job < rows * g.hidden; job += warps) {
        const uint64_t h = job % g.hidden, r = job / g.hidden;
        float routed = 0.0f, shared = 0.0f;
        for (uint64_t p = 0; p < ppr; ++p) {
            const bool is_shared = p == g.topk;
            const uint64_t width = is_shared ? g.shared_inter : g.inter;
            const uint64_t rb = width / dg.elems * dg.bytes;
            const uint8_t *row = is_shared ? (const uint8_t *)w.shared_down + h * rb
                                           : (const uint8_t *)w.down + ((uint64_t)selected[r * g.topk + p] * g.hidden + h) * rb;
            const float *m = mid + (r * ppr + p) * imax;
            float acc = 0.0f;
            for (uint64_t c = lane; c < width; c += 32)
                acc = fmaf(decode_element(g.down_qtype, row + (c / dg.elems) * dg.bytes, (unsigned)(c % dg.elems), status), m[c], acc);
            acc = warp_sum(acc);
            if (!isfinite(acc)) raise(status, YVEX_B200_STATUS_NUMERIC);
            acc = bf16_round(acc);
            if (is_shared) shared = acc; else routed += acc;
        }
        if (lane == 0) {
            out[job] = bf16_round(routed + shared);
            if (routed_out) routed_out[job] = routed;
            if (shared_out) shared_out[job] = shared;
        }
    }
}

}  // namespace yb

using namespace yb;

static int check_geometry(const yvex_b200_moe_geometry *g, const yvex_b200_moe_weights *w) {
    if (!g || !w) return ERR_INVALID_ARG;
    if (!g->hidden || !g->experts || !g->topk || !g->inter || !g->shared_inter) return ERR_INVALID_ARG;
    if (g->experts > 256 || g->topk > 16 || g->topk > g->experts) return ERR_INVALID_ARG;   // src/graph/moe.c:529
    if (g->inter > 4096 || g->shared_inter > 4096) return ERR_BOUNDS;                       // src/graph/moe.c:600
    const unsigned q[3] = {g->gate_qtype, g->up_qtype, g->down_qtype};
    for (unsigned i = 0; i < 3; ++i)
        if (!qtype_supported(q[i])) return ERR_UNSUPPORTED;
    if (g->hidden % geometry_of(g->gate_qtype).elems || g->hidden % geometry_of(g->up_qtype).elems ||
        g->inter % geometry_of(g->down_qtype).elems || g->shared_inter % geometry_of(g->down_qtype).elems)
        return ERR_BOUNDS;
    if (!w->gate || !w->up || !w->down || !w->shared_gate || !w->shared_up || !w->shared_down)
        return ERR_INVALID_ARG;
    if (g->router_class == 0 && (!w->hash_table || !g->hash_rows)) return ERR_INVALID_ARG;
    if (!(g->limit > 0.0) || !isfinite(g->scaling)) return ERR_INVALID_ARG;
    return OK;
}

extern "C" uint64_t yvex_b200_moe_workspace_bytes(const yvex_b200_moe_geometry *g, uint64_t rows) {
    // the fixed part, then the streaming decode path's tables and per-pair rows (narrow batches)
    return g ? moe_decode_stream_layout(*g, rows < 64 ? rows : 64, moe_workspace_layout(*g, rows, nullptr), nullptr) : 0;
}

static int route_into(const MoeGeom &g, const yvex_b200_moe_weights *w, const float *xr,
                      const float *logits_in, const uint32_t *token_ids, uint64_t rows,
                      float *logits_ws, int32_t *selected, float *weights, int *status, cudaStream_t s) {
    const float *logits = logits_in;
    int launches = 1;
    if (w->router) {
        uint64_t jobs = rows * g.experts;
        unsigned grid = grid_for(jobs, 8, 8);
        router_logits_kernel<<<grid, 256, 0, s>>>(w->router, xr, rows, g.experts, g.hidden, logits_ws, status);
        logits = logits_ws;
        ++launches;
    } else if (!logits_in) {
        return ERR_INVALID_ARG;
    }
    route_rows_kernel<<<(unsigned)((rows + 3) / 4), 128, 0, s>>>(g, logits, nullptr, w->bias, w->hash_table, token_ids, rows,
                                                                selected, weights, status, RouteTables{});
    return launch_status(launches);
}

int yb::moe_ingress_and_route(const MoeGeom &g, const MoeWeights &w, const MoeWorkspace &ws, const float *x,
                              const float *logits, const uint32_t *token_ids, uint64_t rows, int *status,
                              cudaStream_t s, RouteTables *tables) {
    const uint64_t n = rows * g.hidden;
    const RouteTables none{};
    if (w.router && rows <= 64 && g.hidden % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0 &&
        (reinterpret_cast<uintptr_t>(w.router) & 15u) == 0) {
        // decode width: two launches (projection with ingress rounding and scoring fused; top-k)
        // both with programmatic stream serialization: launch latency overlaps the kernel before
        if (launch_pdl(ingress_router_kernel, dim3((unsigned)g.experts, (unsigned)rows), dim3(kRouterThreads), 0, s,
                       w.router, x, g.experts, g.hidden, ws.xr, ws.xr_h, ws.logits, ws.scores, status) != cudaSuccess ||
            launch_pdl(route_rows_kernel, dim3((unsigned)((rows + 3) / 4)), dim3(128), 0, s, g, ws.logits, ws.scores, w.bias,
                       w.hash_table, token_ids, rows, ws.selected, ws.weights, status, tables ? *tables : none) != cudaSuccess)
            return ERR_BACKEND;
        return launch_status(2);
    }
    if (tables) tables->enabled = 0;
    ingress_round_kernel<<<grid_for(n, 256, 8), 256, 0, s>>>(x, ws.xr, ws.xr_h, n, status);
    int rc = launch_status(1);
    if (rc != OK) return rc;
    return route_into(g, &w, ws.xr, logits, token_ids, rows, ws.logits, ws.selected, ws.weights, status, s);
}

int yb::moe_check_geometry(const yvex_b200_moe_geometry *g, const yvex_b200_moe_weights *w) {
    return check_geometry(g, w);
}

extern "C" int yvex_b200_moe_route(const yvex_b200_moe_geometry *geom, const yvex_b200_moe_weights *w,
                                   const float *rows_f32, const float *logits, const uint32_t *token_ids,
                                   uint64_t rows, int32_t *selected, float *weights, float *logits_out,
                                   void *workspace, uint64_t workspace_bytes, int *status, void *stream) {
    if (!geom || !w || !selected || !weights || !status || !rows) return ERR_INVALID_ARG;
    if (geom->experts > 256 || geom->topk > 16 || geom->topk > geom->experts || !geom->experts || !geom->topk)
        return ERR_INVALID_ARG;
    MoeGeom g = *geom;
    float *lw = logits_out;
    if (w->router) {
        if (!rows_f32) return ERR_INVALID_ARG;
        if (!lw) {
            if (!workspace || workspace_bytes < rows * g.experts * sizeof(float)) return ERR_NOMEM;
            lw = static_cast<float *>(workspace);
        }
    }
    return route_into(g, w, rows_f32, logits, token_ids, rows, lw, selected, weights, status, as_stream(stream));
}

extern "C" int yvex_b200_moe_ingress(const float *x, uint64_t n, float *rounded_f32, void *rounded_f16, int *status, void *stream) {
    if (!x || !rounded_f32 || !rounded_f16 || !status || !n) return ERR_INVALID_ARG;
    ingress_round_kernel<<<grid_for(n, 256, 8), 256, 0, as_stream(stream)>>>(x, rounded_f32, static_cast<__half *>(rounded_f16), n, status);
    return launch_status(1);
}

extern "C" int yvex_b200_moe_decode(const yvex_b200_moe_geometry *geom, const yvex_b200_moe_weights *w,
                                    const float *x, const float *logits, const uint32_t *token_ids,
                                    uint64_t rows, float *out, int32_t *selected_out, float *weights_out,
                                    void *workspace, uint64_t workspace_bytes, int *status, void *stream) {
    return yvex_b200_moe_decode_parts(geom, w, x, logits, token_ids, rows, out, nullptr, nullptr, selected_out, weights_out, workspace,
                                      workspace_bytes, status, stream);
}

extern "C" int yvex_b200_moe_decode_parts(const yvex_b200_moe_geometry *geom, const yvex_b200_moe_weights *w,
                                          const float *x, const float *logits, const uint32_t *token_ids,
                                          uint64_t rows, float *out, float *routed_out, float *shared_out,
                                          int32_t *selected_out, float *weights_out,
                                          void *workspace, uint64_t workspace_bytes, int *status, void *stream) {
    int rc = check_geometry(geom, w);
    if (rc != OK) return rc;
    if (!x || !out || !status || !rows || rows > 64) return rows > 64 ? ERR_UNSUPPORTED : ERR_INVALID_ARG;
    MoeGeom g = *geom;
    MoeWorkspace ws;
    DecodeStreamScratch stream_scratch;
    const uint64_t fixed = moe_workspace_layout(g, rows, &ws);
    if (!workspace || workspace_bytes < moe_decode_stream_layout(g, rows, fixed, &stream_scratch)) return ERR_NOMEM;
    ws.rebase(workspace);
    stream_scratch.rebase(workspace);
    ws.routed_out = routed_out;
    ws.shared_out = shared_out;
    // the router writes the caller's selection arrays themselves when there are any: no copies behind the layer
    if (selected_out) ws.selected = selected_out;
    if (weights_out) ws.weights = weights_out;
    cudaStream_t s = as_stream(stream);
    mark_phase(0, s);
    const bool streaming = moe_decode_stream_eligible(g, *w);
    RouteTables tables{};
    if (streaming) {
        // the top-k kernel writes the streaming path's matrix tables for its row when it runs at decode width
        const Geometry gg = geometry_of(g.gate_qtype), dg = geometry_of(g.down_qtype);
        tables.w = *w;
        tables.gate_bytes = g.inter * (g.hidden / gg.elems * gg.bytes);
        tables.down_bytes = g.hidden * (g.inter / dg.elems * dg.bytes);
        tables.t = stream_scratch;
        tables.enabled = 1;
    }
    rc = moe_ingress_and_route(g, *w, ws, x, logits, token_ids, rows, status, s, streaming ? &tables : nullptr);
    if (rc != OK) return rc;
    mark_phase(1, s);
    rc = streaming ? moe_experts_stream(g, *w, ws, stream_scratch, tables.enabled != 0, rows, out, status, s)
                   : moe_experts_narrow(g, *w, ws, rows, out, status, s);
    if (rc != OK) return rc;
    return launch_status(0);
}

// Reference-shaped expert execution: used when no streaming decoder covers the layer's qtypes.
int yb::moe_up_rows(const MoeGeom &g, const yvex_b200_moe_weights &w, const MoeWorkspace &ws,
                    uint64_t rows, int *status, cudaStream_t s) {
    const uint64_t imax = g.inter > g.shared_inter ? g.inter : g.shared_inter;
    const uint64_t jobs = rows * (g.topk + 1) * imax;
    expert_up_rows_kernel<<<grid_for(jobs, 8, 16), 256, 0, s>>>(
        g, w, ws.xr, ws.selected, ws.weights, rows, ws.mid, ws.mid_h, status);
    return launch_status(1);
}

int yb::moe_down_rows(const MoeGeom &g, const yvex_b200_moe_weights &w, const MoeWorkspace &ws,
                      uint64_t rows, float *out, int *status, cudaStream_t s) {
    const uint64_t jobs = rows * g.hidden;
    expert_down_rows_kernel<<<grid_for(jobs, 8, 16), 256, 0, s>>>(
        g, w, ws.selected, ws.mid, rows, out, ws.routed_out, ws.shared_out, status);
    return launch_status(1);
}

int yb::moe_experts_rows(const MoeGeom &g, const yvex_b200_moe_weights &w, const MoeWorkspace &ws,
                         uint64_t rows, float *out, int *status, cudaStream_t s) {
    int rc = moe_up_rows(g, w, ws, rows, status, s);
    if (rc != OK) return rc;
    mark_phase(2, s);
    rc = moe_down_rows(g, w, ws, rows, out, status, s);
    mark_phase(3, s);
    return rc;
}
